// Barrier, all-reduce and reduce-scatter over one box's GPUs, each a single kernel.
//
// In a multimem domain every GPU's replica of the payload is bound to one NVSwitch multicast object: one
// `multimem.ld_reduce` returns the sum over all replicas (reduced inside the switch), one `multimem.st` writes all of
// them, one `multimem.red` adds an arrival to every replica's flag. In a peer domain (no multicast) the same kernels
// read and write the members' replicas through plain peer loads and stores in member order.
//
// Rounds live on the device: `flag` only ever grows (arrivals land on every replica), `round` is what this member has
// consumed, so no host write is needed between collectives. A collective enters (every member's data is ready),
// works on its own share, and leaves (every member is done reading), so the kernel's end means the payload is free.
// The payload may be float32 or bfloat16 (reduced in float32); a scale is folded into the store.
//
// Small payloads (up to 64 KiB) have a latency form with ONE arrival round instead of two: every member writes its
// vector into its own slot of a staging area on every replica (one multimem.st per 16 bytes), arrives once, and then
// sums the members' slots from its own replica in member order, so every member computes the same bits. The staging
// area has two sets of slots used alternately (the round's parity), which is what makes the second round unnecessary:
// a set is rewritten only after a later round that every member joined after it had finished reading.
//
// Every wait is bounded: when a member does not show up in time the kernel records status_timeout_collective and
// returns; later collectives on the same domain return at once.
//
// Parity: multimem_barrier_cuda_, multimem_reduce_scatter_cuda_, multimem_all_reduce_cuda_
// (scalingcontrasts.cuh:142-234) and the Mojo peer_* kernels (scalingcontrasts.mojo:604-729).
#include <atomic>
#include <cstdlib>
#include <stdexcept>

#include "api.h"
#include "common.cuh"

namespace sc {

namespace {

constexpr int collective_threads = 512;
constexpr int small_threads = 1024;

// Which form the last collective of this process took: 1 multimem (NVSwitch multicast), 0 peer loads and stores.
std::atomic<int> last_path{-1};

__device__ __forceinline__ void arrive(control_view const& c) {
    if (c.multicast_flag != nullptr) {
        asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(c.multicast_flag), "r"(1u) : "memory");
    } else {
        for (uint32_t peer = 0; peer < c.members; ++peer)
            asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(c.peer_flags[peer]), "r"(1u) : "memory");
    }
}

// Waits until this member's flag has reached `target` (wrap-safe). False when the budget ran out.
__device__ __forceinline__ bool await(control_view const& c, uint32_t target, uint32_t site) {
    uint32_t arrived = 0;
    uint64_t start = 0;
    uint32_t spins = 0;
#pragma unroll 1
    for (;;) {
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(arrived) : "l"(c.own_flag) : "memory");
        if (static_cast<int32_t>(arrived - target) >= 0) return true;
        if ((++spins & 63u) == 0u) {
            uint64_t const now = global_timer_ns();
            if (start == 0) start = now;
            if (now - start > c.budget_ns) {
                record_failure(c.status, status_timeout_collective, site, target, arrived, c.member);
                return false;
            }
        }
    }
}

// Entry of a round. Returns the round in `round`; false when the domain is poisoned or a member never arrived.
__device__ __forceinline__ bool enter(control_view const& c, uint32_t& round) {
    __shared__ uint32_t entered[2];
    if (threadIdx.x == 0) {
        uint32_t const now = *reinterpret_cast<uint32_t volatile*>(c.own_round);
        entered[1] = now;
        bool ok = !status_poisoned(c.status);
        if (ok) {
            if (blockIdx.x == 0) arrive(c);
            ok = await(c, now + c.members, site_collective_enter);
        }
        entered[0] = ok ? 1u : 0u;
    }
    __syncthreads();
    round = entered[1];
    return entered[0] != 0u;
}

// Exit of a round: the last block of this member to finish arrives a second time, waits for every member's last
// block and advances the round by both arrivals.
__device__ __forceinline__ void leave(control_view const& c, uint32_t round) {
    __syncthreads();
    if (threadIdx.x != 0) return;
    __threadfence_system();
    uint32_t previous;
    asm volatile("atom.acq_rel.sys.global.add.u32 %0, [%1], %2;" : "=r"(previous) : "l"(c.own_finished), "r"(1u) : "memory");
    if (previous != gridDim.x - 1) return;
    *reinterpret_cast<uint32_t volatile*>(c.own_finished) = 0u;
    arrive(c);
    if (await(c, round + 2 * c.members, site_collective_leave))
        *reinterpret_cast<uint32_t volatile*>(c.own_round) = round + 2 * c.members;
}

__global__ void barrier_kernel(control_view c) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    if (status_poisoned(c.status)) return;
    uint32_t const round = *reinterpret_cast<uint32_t volatile*>(c.own_round);
    arrive(c);
    if (await(c, round + c.members, site_barrier)) *reinterpret_cast<uint32_t volatile*>(c.own_round) = round + c.members;
}

// Consumes `arrivals` arrivals that this member does not contribute to. With nobody else arriving the wait runs out,
// which is how the timeout path is exercised from the host without faulting anything.
__global__ void expect_arrivals_kernel(control_view c, uint32_t arrivals) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    if (status_poisoned(c.status)) return;
    uint32_t const round = *reinterpret_cast<uint32_t volatile*>(c.own_round);
    if (await(c, round + arrivals, site_barrier)) *reinterpret_cast<uint32_t volatile*>(c.own_round) = round + arrivals;
}

// ---- 16-byte vector primitives -------------------------------------------------------------------------------
struct vec4 {
    uint32_t x, y, z, w;
};

template <payload_type type_>
__device__ __forceinline__ vec4 multimem_load_reduce(void const* multicast_address) {
    vec4 v;
    if constexpr (type_ == payload_type::f32) {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "l"(multicast_address)
                     : "memory");
    } else {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "l"(multicast_address)
                     : "memory");
    }
    return v;
}

template <payload_type type_>
__device__ __forceinline__ void multimem_store(void* multicast_address, vec4 v) {
    if constexpr (type_ == payload_type::f32) {
        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(multicast_address), "r"(v.x),
                     "r"(v.y), "r"(v.z), "r"(v.w)
                     : "memory");
    } else {
        asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(multicast_address),
                     "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                     : "memory");
    }
}

__device__ __forceinline__ vec4 load_vec(void const* address) {
    vec4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(address)
                 : "memory");
    return v;
}
__device__ __forceinline__ void store_vec(void* address, vec4 v) {
    asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(address), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}

__device__ __forceinline__ float2 unpack_bf16x2(uint32_t packed) {
    return make_float2(__uint_as_float(packed << 16), __uint_as_float(packed & 0xFFFF0000u));
}

// Eight (bf16) or four (f32) floats of one vector, so that peer-domain sums and scaling happen in float32.
template <payload_type type_>
struct widened {
    static constexpr int lanes = type_ == payload_type::f32 ? 4 : 8;
    float f[lanes];
    __device__ __forceinline__ static widened from(vec4 v) {
        widened w;
        if constexpr (type_ == payload_type::f32) {
            w.f[0] = __uint_as_float(v.x), w.f[1] = __uint_as_float(v.y), w.f[2] = __uint_as_float(v.z),
            w.f[3] = __uint_as_float(v.w);
        } else {
            float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
            w.f[0] = a.x, w.f[1] = a.y, w.f[2] = b.x, w.f[3] = b.y, w.f[4] = c.x, w.f[5] = c.y, w.f[6] = d.x, w.f[7] = d.y;
        }
        return w;
    }
    __device__ __forceinline__ vec4 narrow() const {
        vec4 v;
        if constexpr (type_ == payload_type::f32) {
            v.x = __float_as_uint(f[0]), v.y = __float_as_uint(f[1]), v.z = __float_as_uint(f[2]),
            v.w = __float_as_uint(f[3]);
        } else {
            v.x = pack_bf16x2(f[0], f[1]), v.y = pack_bf16x2(f[2], f[3]), v.z = pack_bf16x2(f[4], f[5]),
            v.w = pack_bf16x2(f[6], f[7]);
        }
        return v;
    }
    __device__ __forceinline__ void scale(float s) {
#pragma unroll
        for (int i = 0; i < lanes; ++i) f[i] *= s;
    }
    __device__ __forceinline__ void add(widened const& o) {
#pragma unroll
        for (int i = 0; i < lanes; ++i) f[i] += o.f[i];
    }
};

struct replica_list {
    void* at[16];
};

// The sum over members of vector `index`, reduced in the switch (multicast) or by peer loads in member order.
template <payload_type type_, bool multicast_>
__device__ __forceinline__ vec4 reduce_vector(control_view const& c, char* multicast, replica_list const& replicas,
                                              size_t byte_offset, float scale) {
    if constexpr (multicast_) {
        vec4 v = multimem_load_reduce<type_>(multicast + byte_offset);
        if (scale != 1.0f) {
            widened<type_> w = widened<type_>::from(v);
            w.scale(scale);
            v = w.narrow();
        }
        return v;
    } else {
        widened<type_> total = widened<type_>::from(load_vec(static_cast<char*>(replicas.at[0]) + byte_offset));
        for (uint32_t peer = 1; peer < c.members; ++peer)
            total.add(widened<type_>::from(load_vec(static_cast<char*>(replicas.at[peer]) + byte_offset)));
        if (scale != 1.0f) total.scale(scale);
        return total.narrow();
    }
}

template <payload_type type_, bool multicast_, int collective_unroll>
__global__ void __launch_bounds__(collective_threads)
    all_reduce_kernel(control_view c, char* multicast, replica_list replicas, size_t first_vector, size_t vectors,
                      float scale) {
    uint32_t round;
    if (!enter(c, round)) return;
    size_t const share = (vectors + c.members - 1) / c.members;
    size_t const begin = min(static_cast<size_t>(c.member) * share, vectors);
    size_t const end = min(begin + share, vectors);
    size_t const stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t base = begin + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; base < end;
         base += stride * collective_unroll) {
        vec4 v[collective_unroll];
#pragma unroll
        for (int u = 0; u < collective_unroll; ++u) {
            size_t const index = base + u * stride;
            if (index < end) v[u] = reduce_vector<type_, multicast_>(c, multicast, replicas, (first_vector + index) * 16, scale);
        }
#pragma unroll
        for (int u = 0; u < collective_unroll; ++u) {
            size_t const index = base + u * stride;
            if (index >= end) continue;
            size_t const offset = (first_vector + index) * 16;
            if constexpr (multicast_) {
                multimem_store<type_>(multicast + offset, v[u]);
            } else {
                for (uint32_t peer = 0; peer < c.members; ++peer) store_vec(static_cast<char*>(replicas.at[peer]) + offset, v[u]);
            }
        }
    }
    leave(c, round);
}

template <payload_type type_, bool multicast_, int collective_unroll>
__global__ void __launch_bounds__(collective_threads)
    reduce_scatter_kernel(control_view c, char* multicast, replica_list replicas, char* own, size_t first_vector,
                          size_t shard_vectors, float scale, float* out_f32) {
    uint32_t round;
    if (!enter(c, round)) return;
    size_t const begin = static_cast<size_t>(c.member) * shard_vectors;
    size_t const end = begin + shard_vectors;
    size_t const stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t base = begin + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; base < end;
         base += stride * collective_unroll) {
        vec4 v[collective_unroll];
#pragma unroll
        for (int u = 0; u < collective_unroll; ++u) {
            size_t const index = base + u * stride;
            if (index < end)
                v[u] = reduce_vector<type_, multicast_>(c, multicast, replicas, (first_vector + index) * 16,
                                                        out_f32 == nullptr ? scale : 1.0f);
        }
#pragma unroll
        for (int u = 0; u < collective_unroll; ++u) {
            size_t const index = base + u * stride;
            if (index >= end) continue;
            if (out_f32 == nullptr) {
                store_vec(own + (first_vector + index) * 16, v[u]);
            } else {
                widened<type_> w = widened<type_>::from(v[u]);
                w.scale(scale);
                float* destination = out_f32 + (index - begin) * widened<type_>::lanes;
#pragma unroll
                for (int i = 0; i < widened<type_>::lanes; i += 4)
                    *reinterpret_cast<float4*>(destination + i) = make_float4(w.f[i], w.f[i + 1], w.f[i + 2], w.f[i + 3]);
            }
        }
    }
    leave(c, round);
}

// The latency form for small payloads: one block, one arrival round. `own_payload` is this member's payload (read, then
// overwritten with the sum), `slots` the staging area as seen through the multicast alias (or null), `slot_replicas`
// every member's staging area (peer form), `own_slots` this member's. Slot (parity, member) starts at
// (parity * members + member) * slot_bytes.
template <payload_type type_, bool multicast_>
__global__ void __launch_bounds__(small_threads)
    all_reduce_small_kernel(control_view c, char* own_payload, char* slots, replica_list slot_replicas, char* own_slots,
                            uint32_t vectors, uint32_t slot_bytes, float scale) {
    __shared__ uint32_t shared_round, shared_ok;
    if (threadIdx.x == 0) {
        shared_round = *reinterpret_cast<uint32_t volatile*>(c.own_round);
        shared_ok = status_poisoned(c.status) ? 0u : 1u;
    }
    __syncthreads();
    if (shared_ok == 0u) return;
    uint32_t const round = shared_round;
    uint32_t const parity = (round / c.members) & 1u;
    size_t const mine = static_cast<size_t>(parity * c.members + c.member) * slot_bytes;
    for (uint32_t v = threadIdx.x; v < vectors; v += blockDim.x) {
        if (!SC_IN_BOUNDS(static_cast<size_t>(v) * 16 + 15, slot_bytes)) continue;
        vec4 const value = load_vec(own_payload + static_cast<size_t>(v) * 16);
        if constexpr (multicast_) {
            multimem_store<payload_type::f32>(slots + mine + static_cast<size_t>(v) * 16, value);
        } else {
            for (uint32_t peer = 0; peer < c.members; ++peer)
                store_vec(static_cast<char*>(slot_replicas.at[peer]) + mine + static_cast<size_t>(v) * 16, value);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        arrive(c);
        bool const ok = await(c, round + c.members, site_collective_enter);
        if (ok) *reinterpret_cast<uint32_t volatile*>(c.own_round) = round + c.members;
        shared_ok = ok ? 1u : 0u;
    }
    __syncthreads();
    if (shared_ok == 0u) return;
    char const* const first = own_slots + static_cast<size_t>(parity * c.members) * slot_bytes;
    for (uint32_t v = threadIdx.x; v < vectors; v += blockDim.x) {
        widened<type_> total = widened<type_>::from(load_vec(first + static_cast<size_t>(v) * 16));
        for (uint32_t peer = 1; peer < c.members; ++peer)
            total.add(widened<type_>::from(load_vec(first + static_cast<size_t>(peer) * slot_bytes + static_cast<size_t>(v) * 16)));
        if (scale != 1.0f) total.scale(scale);
        store_vec(own_payload + static_cast<size_t>(v) * 16, total.narrow());
    }
}

// How a bandwidth-class collective is cut: vectors in flight per thread (1, 2, 4 or 8) and the number of blocks (one per
// multiprocessor at most). Measured: spreading a member's share over more blocks beats more vectors in flight per thread at
// every size (2 GPUs, 16 MiB all-reduce: 64.4 us with 2 per thread, 67.0 with 4, 67.8 with 8; 128 MiB: 359 / 372 / 389 us;
// 64 blocks instead of 148 cost a reduce-scatter of 128 MiB 40 %), so a share that fits one vector per thread of a full
// grid takes one, anything larger two. Both can be forced from the environment (SC_COLLECTIVE_UNROLL,
// SC_COLLECTIVE_MAX_BLOCKS) to sweep them.
struct shape_t {
    int unroll, blocks;
};
shape_t shape_for(size_t vectors, int multiprocessors) {
    static int const forced_unroll = std::getenv("SC_COLLECTIVE_UNROLL") ? std::atoi(std::getenv("SC_COLLECTIVE_UNROLL")) : 0;
    static int const forced_blocks = std::getenv("SC_COLLECTIVE_MAX_BLOCKS") ? std::atoi(std::getenv("SC_COLLECTIVE_MAX_BLOCKS")) : 0;
    int const cap = forced_blocks > 0 ? forced_blocks : multiprocessors;
    int unroll = vectors <= static_cast<size_t>(cap) * collective_threads ? 1 : 2;
    if (forced_unroll == 1 || forced_unroll == 2 || forced_unroll == 4 || forced_unroll == 8) unroll = forced_unroll;
    size_t const per_block = static_cast<size_t>(collective_threads) * unroll;
    size_t blocks = (vectors + per_block - 1) / per_block;
    if (blocks < 1) blocks = 1;
    if (blocks > static_cast<size_t>(cap)) blocks = static_cast<size_t>(cap);
    return shape_t{unroll, static_cast<int>(blocks)};
}

void check_launch(char const* what) {
    cudaError_t const error = cudaGetLastError();
    if (error != cudaSuccess) throw std::runtime_error(std::string(what) + " launch failed: " + cudaGetErrorString(error));
    note_launch();
}

replica_list make_list(control_view const& control, void* const* replicas) {
    replica_list list{};
    if (replicas != nullptr)
        for (uint32_t i = 0; i < control.members && i < 16; ++i) list.at[i] = replicas[i];
    return list;
}

size_t vector_scalars(payload_type type) { return type == payload_type::f32 ? 4 : 8; }

template <payload_type type_, bool multicast_>
void launch_all_reduce_shape(shape_t shape, control_view const& control, char* mc, replica_list const& list, size_t first_vector,
                             size_t vectors, float scale, cudaStream_t stream) {
    if (shape.unroll == 1)
        all_reduce_kernel<type_, multicast_, 1><<<shape.blocks, collective_threads, 0, stream>>>(control, mc, list, first_vector, vectors, scale);
    else if (shape.unroll == 2)
        all_reduce_kernel<type_, multicast_, 2><<<shape.blocks, collective_threads, 0, stream>>>(control, mc, list, first_vector, vectors, scale);
    else if (shape.unroll == 8)
        all_reduce_kernel<type_, multicast_, 8><<<shape.blocks, collective_threads, 0, stream>>>(control, mc, list, first_vector, vectors, scale);
    else
        all_reduce_kernel<type_, multicast_, 4><<<shape.blocks, collective_threads, 0, stream>>>(control, mc, list, first_vector, vectors, scale);
}
template <payload_type type_, bool multicast_>
void launch_reduce_scatter_shape(shape_t shape, control_view const& control, char* mc, replica_list const& list, char* mine,
                                 size_t first_vector, size_t shard_vectors, float scale, float* out_f32, cudaStream_t stream) {
    if (shape.unroll == 1)
        reduce_scatter_kernel<type_, multicast_, 1><<<shape.blocks, collective_threads, 0, stream>>>(control, mc, list, mine, first_vector, shard_vectors, scale, out_f32);
    else if (shape.unroll == 2)
        reduce_scatter_kernel<type_, multicast_, 2><<<shape.blocks, collective_threads, 0, stream>>>(control, mc, list, mine, first_vector, shard_vectors, scale, out_f32);
    else if (shape.unroll == 8)
        reduce_scatter_kernel<type_, multicast_, 8><<<shape.blocks, collective_threads, 0, stream>>>(control, mc, list, mine, first_vector, shard_vectors, scale, out_f32);
    else
        reduce_scatter_kernel<type_, multicast_, 4><<<shape.blocks, collective_threads, 0, stream>>>(control, mc, list, mine, first_vector, shard_vectors, scale, out_f32);
}

} // namespace

int last_collective_path() { return last_path.load(); }
SC_DEFINE_BOUNDS_READER(bounds_record_collectives)

void launch_barrier(control_view const& control, cudaStream_t stream) {
    barrier_kernel<<<1, 32, 0, stream>>>(control);
    check_launch("barrier");
    last_path.store(control.multicast_flag != nullptr ? 1 : 0);
}

void launch_expect_arrivals(control_view const& control, uint32_t arrivals, cudaStream_t stream) {
    expect_arrivals_kernel<<<1, 32, 0, stream>>>(control, arrivals);
    check_launch("expect_arrivals");
}

void launch_all_reduce(control_view const& control, void* multicast, void* const* replicas, size_t first, size_t scalars,
                       payload_type type, float scale, int multiprocessors, cudaStream_t stream) {
    size_t const per_vector = vector_scalars(type);
    if (first % per_vector || scalars % per_vector)
        throw std::runtime_error("all_reduce: offset and size must be multiples of one 16-byte vector");
    if (control.members > 16) throw std::runtime_error("all_reduce: at most 16 members");
    size_t const vectors = scalars / per_vector, first_vector = first / per_vector;
    size_t const share = (vectors + control.members - 1) / control.members;
    shape_t const shape = shape_for(share, multiprocessors);
    replica_list const list = make_list(control, replicas);
    char* const mc = static_cast<char*>(multicast);
    bool const multicast_path = multicast != nullptr && control.multicast_flag != nullptr;
    if (type == payload_type::f32) {
        if (multicast_path) launch_all_reduce_shape<payload_type::f32, true>(shape, control, mc, list, first_vector, vectors, scale, stream);
        else launch_all_reduce_shape<payload_type::f32, false>(shape, control, mc, list, first_vector, vectors, scale, stream);
    } else {
        if (multicast_path) launch_all_reduce_shape<payload_type::bf16, true>(shape, control, mc, list, first_vector, vectors, scale, stream);
        else launch_all_reduce_shape<payload_type::bf16, false>(shape, control, mc, list, first_vector, vectors, scale, stream);
    }
    check_launch("all_reduce");
    last_path.store(multicast_path ? 1 : 0);
}

void launch_all_reduce_small(control_view const& control, void* own_payload, void* multicast_slots, void* const* slot_replicas,
                             void* own_slots, size_t scalars, payload_type type, float scale, size_t slot_bytes,
                             cudaStream_t stream) {
    size_t const per_vector = vector_scalars(type);
    if (scalars == 0 || scalars % per_vector) throw std::runtime_error("all_reduce_small: size must be a multiple of one 16-byte vector");
    size_t const vectors = scalars / per_vector;
    if (vectors * 16 > slot_bytes || slot_bytes % 16) throw std::runtime_error("all_reduce_small: the payload does not fit a staging slot");
    if (control.members > 16) throw std::runtime_error("all_reduce_small: at most 16 members");
    if (own_payload == nullptr || own_slots == nullptr) throw std::runtime_error("all_reduce_small: missing payload or staging area");
    replica_list const list = make_list(control, slot_replicas);
    bool const multicast_path = multicast_slots != nullptr && control.multicast_flag != nullptr;
    int const threads = vectors >= small_threads ? small_threads : static_cast<int>((vectors + 31) / 32 * 32);
    char* const payload = static_cast<char*>(own_payload);
    char* const mc = static_cast<char*>(multicast_slots);
    char* const mine = static_cast<char*>(own_slots);
    uint32_t const v = static_cast<uint32_t>(vectors), bytes = static_cast<uint32_t>(slot_bytes);
    if (type == payload_type::f32) {
        if (multicast_path) all_reduce_small_kernel<payload_type::f32, true><<<1, threads, 0, stream>>>(control, payload, mc, list, mine, v, bytes, scale);
        else all_reduce_small_kernel<payload_type::f32, false><<<1, threads, 0, stream>>>(control, payload, mc, list, mine, v, bytes, scale);
    } else {
        if (multicast_path) all_reduce_small_kernel<payload_type::bf16, true><<<1, threads, 0, stream>>>(control, payload, mc, list, mine, v, bytes, scale);
        else all_reduce_small_kernel<payload_type::bf16, false><<<1, threads, 0, stream>>>(control, payload, mc, list, mine, v, bytes, scale);
    }
    check_launch("all_reduce_small");
    last_path.store(multicast_path ? 1 : 0);
}

void launch_reduce_scatter(control_view const& control, void* multicast, void* const* replicas, void* own, size_t first,
                           size_t shard_scalars, payload_type type, float scale, float* out_f32, int multiprocessors,
                           cudaStream_t stream) {
    size_t const per_vector = vector_scalars(type);
    if (first % per_vector || shard_scalars % per_vector)
        throw std::runtime_error("reduce_scatter: offset and shard must be multiples of one 16-byte vector");
    if (control.members > 16) throw std::runtime_error("reduce_scatter: at most 16 members");
    size_t const shard_vectors = shard_scalars / per_vector, first_vector = first / per_vector;
    shape_t const shape = shape_for(shard_vectors, multiprocessors);
    replica_list const list = make_list(control, replicas);
    char* const mc = static_cast<char*>(multicast);
    char* const mine = static_cast<char*>(own);
    bool const multicast_path = multicast != nullptr && control.multicast_flag != nullptr;
    if (type == payload_type::f32) {
        if (multicast_path) launch_reduce_scatter_shape<payload_type::f32, true>(shape, control, mc, list, mine, first_vector, shard_vectors, scale, out_f32, stream);
        else launch_reduce_scatter_shape<payload_type::f32, false>(shape, control, mc, list, mine, first_vector, shard_vectors, scale, out_f32, stream);
    } else {
        if (multicast_path) launch_reduce_scatter_shape<payload_type::bf16, true>(shape, control, mc, list, mine, first_vector, shard_vectors, scale, out_f32, stream);
        else launch_reduce_scatter_shape<payload_type::bf16, false>(shape, control, mc, list, mine, first_vector, shard_vectors, scale, out_f32, stream);
    }
    check_launch("reduce_scatter");
    last_path.store(multicast_path ? 1 : 0);
}

// Loads every collective kernel's code onto the current device while it is idle. A first launch that has to load its
// module can wait for the device to go idle, which a peer spinning in a collective never lets happen.
void preload_collective_kernels() {
    cudaFuncAttributes attributes;
    auto touch = [&](void const* function) {
        cudaError_t const error = cudaFuncGetAttributes(&attributes, function);
        if (error != cudaSuccess) throw std::runtime_error(std::string("preload failed: ") + cudaGetErrorString(error));
    };
    touch(reinterpret_cast<void const*>(&barrier_kernel));
    touch(reinterpret_cast<void const*>(&expect_arrivals_kernel));
#define SC_TOUCH_SHAPES(kernel)                                                                                          \
    touch(reinterpret_cast<void const*>(&kernel<payload_type::f32, true, 1>));                                           \
    touch(reinterpret_cast<void const*>(&kernel<payload_type::f32, false, 1>));                                          \
    touch(reinterpret_cast<void const*>(&kernel<payload_type::bf16, true, 1>));                                          \
    touch(reinterpret_cast<void const*>(&kernel<payload_type::bf16, false, 1>));                                         \
    touch(reinterpret_cast<void const*>(&kernel<payload_type::f32, true, 2>));                                           \
    touch(reinterpret_cast<void const*>(&kernel<payload_type::f32, true, 4>));                                           \
    touch(reinterpret_cast<void const*>(&kernel<payload_type::f32, true, 8>));                                           \
    touch(reinterpret_cast<void const*>(&kernel<payload_type::f32, false, 2>));                                          \
    touch(reinterpret_cast<void const*>(&kernel<payload_type::f32, false, 4>));                                          \
    touch(reinterpret_cast<void const*>(&kernel<payload_type::f32, false, 8>));                                          \
    touch(reinterpret_cast<void const*>(&kernel<payload_type::bf16, true, 2>));                                          \
    touch(reinterpret_cast<void const*>(&kernel<payload_type::bf16, true, 4>));                                          \
    touch(reinterpret_cast<void const*>(&kernel<payload_type::bf16, true, 8>));                                          \
    touch(reinterpret_cast<void const*>(&kernel<payload_type::bf16, false, 2>));                                         \
    touch(reinterpret_cast<void const*>(&kernel<payload_type::bf16, false, 4>));                                         \
    touch(reinterpret_cast<void const*>(&kernel<payload_type::bf16, false, 8>));
    SC_TOUCH_SHAPES(all_reduce_kernel)
    SC_TOUCH_SHAPES(reduce_scatter_kernel)
#undef SC_TOUCH_SHAPES
    touch(reinterpret_cast<void const*>(&all_reduce_small_kernel<payload_type::f32, true>));
    touch(reinterpret_cast<void const*>(&all_reduce_small_kernel<payload_type::f32, false>));
    touch(reinterpret_cast<void const*>(&all_reduce_small_kernel<payload_type::bf16, true>));
    touch(reinterpret_cast<void const*>(&all_reduce_small_kernel<payload_type::bf16, false>));
}

} // namespace sc
