// Shared device-side helpers for the sm_100a kernels: status words, bounded waits, mbarrier / TMA / tcgen05 wrappers.
//
// Every wait in this library is bounded. A wait that runs out records where and why in a status block that the host
// reads, raises the CTA's abort flag so that the other warps stop waiting too, and returns; the kernel then frees its
// tensor memory and ends. Nothing here traps, asserts or spins without a limit: the GPUs are shared.
//
// Parity: these cover the reference's L2 layer (scalingcontrasts.cuh:142-184 multimem arrive/await, :717-843 mbarrier,
// TMA and tcgen05 wrappers), whose waits are unbounded.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace sc {

// ---------------------------------------------------------------------------------------------------------------
// Status block: eight 32-bit words in device (or symmetric) memory. Word 0 is the code; it is sticky: the first
// failure wins and every later kernel that is given the block returns at once while it is non-zero.
// ---------------------------------------------------------------------------------------------------------------
enum status_code : uint32_t {
    status_ok = 0,
    status_timeout_collective = 1, // a member did not arrive within the budget
    status_timeout_pipeline = 2,   // an mbarrier inside a tile kernel did not complete within the budget
    status_bad_argument = 3,
};
constexpr int status_words = 8;

// Sites, so that a timeout names the wait that ran out.
enum wait_site : uint32_t {
    site_collective_enter = 1,
    site_collective_leave = 2,
    site_barrier = 3,
    site_fwd_stage_full = 10,
    site_fwd_stage_empty = 11,
    site_fwd_slot_empty = 12,
    site_fwd_tile_full = 13,
    site_bwd_stage_full = 20,
    site_bwd_stage_empty = 21,
    site_bwd_accumulated = 22,
    site_drain = 30,
    site_fz_item_stored = 40,
    site_fz_stage_empty = 41,
    site_fz_stage_full = 42,
    site_fz_accumulator_empty = 43,
    site_fz_accumulator_full = 44,
};

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void record_failure(uint32_t* status, uint32_t code, uint32_t site, uint32_t a, uint32_t b,
                                               uint32_t c) {
    if (status == nullptr) return;
    if (atomicCAS(status, 0u, code) == 0u) {
        status[1] = site;
        status[2] = a;
        status[3] = b;
        status[4] = c;
        status[5] = blockIdx.x;
        status[6] = threadIdx.x;
        __threadfence_system();
    }
}

__device__ __forceinline__ bool status_poisoned(uint32_t const* status) {
    return status != nullptr && *reinterpret_cast<uint32_t const volatile*>(status) != 0u;
}

// ---------------------------------------------------------------------------------------------------------------
// Bounds-checked debug build (-DSC_BOUNDS=1): every index into global memory that a kernel computes is compared with
// its limit first. A miss is recorded (first one wins: code, source line, index, limit, block, thread) in a record that
// the host reads, and the access is skipped; nothing traps. In the ordinary build the check compiles to `true`. The
// record lives once per translation unit; SC_DEFINE_BOUNDS_READER gives the unit a host function that copies it out.
// ---------------------------------------------------------------------------------------------------------------
#ifndef SC_BOUNDS
#define SC_BOUNDS 0
#endif
#if SC_BOUNDS
static __device__ uint32_t bounds_record[8];
__device__ __forceinline__ bool in_bounds(uint64_t index, uint64_t limit, uint32_t line) {
    if (index < limit) return true;
    if (atomicCAS(&bounds_record[0], 0u, static_cast<uint32_t>(status_bad_argument)) == 0u) {
        bounds_record[1] = line;
        bounds_record[2] = static_cast<uint32_t>(index), bounds_record[3] = static_cast<uint32_t>(index >> 32);
        bounds_record[4] = static_cast<uint32_t>(limit), bounds_record[5] = static_cast<uint32_t>(limit >> 32);
        bounds_record[6] = blockIdx.x, bounds_record[7] = threadIdx.x;
    }
    return false;
}
#define SC_IN_BOUNDS(index, limit) ::sc::in_bounds(static_cast<uint64_t>(index), static_cast<uint64_t>(limit), __LINE__)
// The same for a whole converged warp in front of a warp-wide instruction: all lanes pass or all lanes skip.
#define SC_WARP_IN_BOUNDS(index, limit) __all_sync(0xFFFFFFFFu, SC_IN_BOUNDS(index, limit))
#define SC_DEFINE_BOUNDS_READER(name)                                                                                   \
    void name(uint32_t* out) {                                                                                          \
        if (cudaMemcpyFromSymbol(out, bounds_record, sizeof(bounds_record)) != cudaSuccess)                             \
            for (int i = 0; i < 8; ++i) out[i] = 0xFFFFFFFFu;                                                           \
    }
#else
#define SC_IN_BOUNDS(index, limit) true
#define SC_WARP_IN_BOUNDS(index, limit) true
#define SC_DEFINE_BOUNDS_READER(name)                                                                                   \
    void name(uint32_t* out) {                                                                                          \
        for (int i = 0; i < 8; ++i) out[i] = 0u;                                                                        \
    }
#endif

// ---------------------------------------------------------------------------------------------------------------
// Shared-memory addresses and mbarriers
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(void const* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One attempt: the thread may be suspended until the phase completes or the hinted time has passed, whichever is first.
// The hint keeps a waiting warp from burning issue slots on retries; it does not delay the wake-up on completion.
constexpr uint32_t mbar_suspend_hint_ns = 20000;
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(mbar_suspend_hint_ns)
        : "memory");
    return done != 0;
}
// One attempt that never suspends: has the phase with this parity completed?
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// The same for every state space: orders this thread's view of global memory written by bulk stores with bulk loads
// that another thread issues after it has been told (through an mbarrier) that the stores are complete.
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// The context a bounded wait needs: where to report, how long to wait, and the CTA's abort flag in shared memory.
struct wait_context {
    uint32_t* status;
    uint64_t budget_ns;
    uint32_t volatile* abort_flag; // shared memory, one per CTA
};

// Waits for the phase with the given parity to complete. Returns false when the budget ran out or when another warp of
// the CTA has already given up; in the first case the failure is recorded and the abort flag raised. The common case (the
// phase completes within a few attempts) is inlined; the timed part is one real call, so that a kernel with a dozen waits
// carries its code once.
static __device__ __noinline__ bool mbar_wait_timed(uint32_t bar, uint32_t parity, uint32_t* status, uint64_t budget_ns,
                                             uint32_t volatile* abort_flag, uint32_t site, uint32_t detail) {
    uint64_t const start = global_timer_ns();
#pragma unroll 1
    for (;;) {
#pragma unroll 1
        for (int spin = 0; spin < 64; ++spin)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag != 0u) return false;
        if (global_timer_ns() - start > budget_ns) {
            record_failure(status, status_timeout_pipeline, site, detail, parity, bar);
            *abort_flag = 1u;
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, wait_context const& ctx, uint32_t site,
                                          uint32_t detail) {
#pragma unroll 1
    for (int spin = 0; spin < 16; ++spin)
        if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_timed(bar, parity, ctx.status, ctx.budget_ns, ctx.abort_flag, site, detail);
}

// The same wait for a helper warp that shares its scheduler with warps doing arithmetic: between attempts it sleeps, so
// that its polling does not take issue slots from them. The price is up to `sleep_ns` of wake-up latency, which suits
// waits that have slack (a producer ahead of its consumer) and not those on a critical path.
static __device__ __noinline__ bool mbar_wait_sleeping(uint32_t bar, uint32_t parity, uint32_t* status, uint64_t budget_ns,
                                                       uint32_t volatile* abort_flag, uint32_t site, uint32_t detail,
                                                       uint32_t sleep_ns) {
    uint64_t const start = global_timer_ns();
#pragma unroll 1
    for (;;) {
#pragma unroll 1
        for (int spin = 0; spin < 64; ++spin) {
            __nanosleep(sleep_ns);
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (*abort_flag != 0u) return false;
        if (global_timer_ns() - start > budget_ns) {
            record_failure(status, status_timeout_pipeline, site, detail, parity, bar);
            *abort_flag = 1u;
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, wait_context const& ctx, uint32_t site,
                                                  uint32_t detail, uint32_t sleep_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_sleeping(bar, parity, ctx.status, ctx.budget_ns, ctx.abort_flag, site, detail, sleep_ns);
}

// ---------------------------------------------------------------------------------------------------------------
// TMA: tiled bulk tensor loads into this CTA's shared memory, completion counted on an mbarrier. No load in this
// library carries a cluster multicast qualifier, and no tensor map covers another GPU's memory.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_descriptor(CUtensorMap const* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, CUtensorMap const* map, uint32_t bar, int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, CUtensorMap const* map, uint32_t bar, int32_t x, int32_t y,
                                            int32_t z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
// tcgen05: tensor memory allocation, UMMA issue, commit, loads
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t result_slot_smem, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_slot_smem), "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], bf16 inputs, fp32 accumulate. `accumulate` == 0 overwrites D.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One lane of a converged warp, chosen by the hardware. Roles that issue TMA or UMMA instructions run warp-wide and put
// only those instructions under this predicate, so that their operands stay warp-uniform values.
__device__ __forceinline__ bool elect_one() {
    uint32_t elected;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(elected));
    return elected != 0u;
}
// Makes the mbarrier track the completion of every UMMA this thread issued before it.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Shared-memory matrix descriptor for a K-major bf16 operand stored as rows of 64 elements (128 bytes) under the
// 128-byte swizzle: eight rows make one 1024-byte atom, atoms follow one another every `stride_bytes` (1024 when rows
// are dense). Stepping 16 elements along K inside the row adds 32 bytes to the start address.
__device__ __forceinline__ uint64_t umma_desc_k_major_sw128(uint32_t smem_address, uint32_t stride_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_address & 0x3FFFFu) >> 4);        // bits 0-13: start address / 16
    d |= static_cast<uint64_t>(1) << 16;                                // bits 16-29: leading offset (unused here) = 1
    d |= static_cast<uint64_t>((stride_bytes >> 4) & 0x3FFFu) << 32;    // bits 32-45: stride between 8-row atoms / 16
    d |= static_cast<uint64_t>(1) << 46;                                // bits 46-48: descriptor version 1
    d |= static_cast<uint64_t>(2) << 61;                                // bits 61-63: 128-byte swizzle
    return d;
}

// Instruction descriptor: fp32 accumulator, bf16 A and B, both K-major, tile M x N.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(uint32_t m, uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Bit that marks the B operand as MN-major (its N dimension is the contiguous one in shared memory) instead of K-major.
constexpr uint32_t umma_idesc_b_mn_major = 1u << 16;

// 32 lanes x 16 consecutive columns of 32-bit values: thread t of the warp gets lane (base lane + t).
__device__ __forceinline__ void tmem_load_16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------------------------
// Small arithmetic helpers
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float fast_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// log1p(x) / x on [0, 1] as a degree-8 polynomial: a Remez exchange fit of the relative error made for this library
// (3.0e-8 in exact arithmetic, 2.1e-7 when evaluated in float32 by Horner's rule over two million points).
#define SC_LOG1P_C0 9.999999404e-01f
#define SC_LOG1P_C1 -4.999949336e-01f
#define SC_LOG1P_C2 3.331909776e-01f
#define SC_LOG1P_C3 -2.484298199e-01f
#define SC_LOG1P_C4 1.910600662e-01f
#define SC_LOG1P_C5 -1.366324574e-01f
#define SC_LOG1P_C6 7.822595537e-02f
#define SC_LOG1P_C7 -2.950523980e-02f
#define SC_LOG1P_C8 5.232694093e-03f
__device__ __forceinline__ float log1p_unit(float x) {
    float p = SC_LOG1P_C8;
    p = fmaf(p, x, SC_LOG1P_C7);
    p = fmaf(p, x, SC_LOG1P_C6);
    p = fmaf(p, x, SC_LOG1P_C5);
    p = fmaf(p, x, SC_LOG1P_C4);
    p = fmaf(p, x, SC_LOG1P_C3);
    p = fmaf(p, x, SC_LOG1P_C2);
    p = fmaf(p, x, SC_LOG1P_C1);
    p = fmaf(p, x, SC_LOG1P_C0);
    return p * x;
}
// The polynomial alone: log1p(x) = log1p_ratio(x) * x, for callers that fold the product into an accumulation.
__device__ __forceinline__ float log1p_ratio(float x) {
    float p = SC_LOG1P_C8;
    p = fmaf(p, x, SC_LOG1P_C7);
    p = fmaf(p, x, SC_LOG1P_C6);
    p = fmaf(p, x, SC_LOG1P_C5);
    p = fmaf(p, x, SC_LOG1P_C4);
    p = fmaf(p, x, SC_LOG1P_C3);
    p = fmaf(p, x, SC_LOG1P_C2);
    p = fmaf(p, x, SC_LOG1P_C1);
    return fmaf(p, x, SC_LOG1P_C0);
}

// Packed pairs of float32 in one 64-bit register: sm_100 executes add / mul / fma on both halves in one instruction,
// which halves the issue slots of the epilogue's arithmetic. The compiler's own float2 intrinsics are used (not opaque
// inline assembly), so it can keep the halves where the scalar instructions around them (MUFU, tensor-memory loads and
// stores) want them and fold sign changes into operands.
using pair_t = float2;
__device__ __forceinline__ pair_t pack2(float lo, float hi) { return make_float2(lo, hi); }
__device__ __forceinline__ void unpack2(pair_t v, float& lo, float& hi) { lo = v.x, hi = v.y; }
__device__ __forceinline__ pair_t add2(pair_t a, pair_t b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ pair_t mul2(pair_t a, pair_t b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ pair_t fma2(pair_t a, pair_t b, pair_t c) { return __ffma2_rn(a, b, c); }
// log1p(x) / x for both halves of a pair (the same polynomial as log1p_ratio). The coefficients sit in constant memory
// already duplicated into pairs, so that they can be operands of the packed instructions without register pairs of
// their own.
__constant__ float2 log1p_pairs[9] = {{SC_LOG1P_C0, SC_LOG1P_C0}, {SC_LOG1P_C1, SC_LOG1P_C1}, {SC_LOG1P_C2, SC_LOG1P_C2},
                                      {SC_LOG1P_C3, SC_LOG1P_C3}, {SC_LOG1P_C4, SC_LOG1P_C4}, {SC_LOG1P_C5, SC_LOG1P_C5},
                                      {SC_LOG1P_C6, SC_LOG1P_C6}, {SC_LOG1P_C7, SC_LOG1P_C7}, {SC_LOG1P_C8, SC_LOG1P_C8}};
__device__ __forceinline__ pair_t log1p_pair(int index) { return log1p_pairs[index]; }
__device__ __forceinline__ pair_t log1p_ratio2(pair_t x) {
    pair_t p = log1p_pair(8);
    p = fma2(p, x, log1p_pair(7));
    p = fma2(p, x, log1p_pair(6));
    p = fma2(p, x, log1p_pair(5));
    p = fma2(p, x, log1p_pair(4));
    p = fma2(p, x, log1p_pair(3));
    p = fma2(p, x, log1p_pair(2));
    p = fma2(p, x, log1p_pair(1));
    return fma2(p, x, log1p_pair(0));
}

// Matryoshka ladder by value, the form kernels take (ascending ends, zero padded).
struct ladder_t {
    uint32_t count;
    uint32_t ends[8];
    __host__ __device__ uint32_t begin(uint32_t band) const { return band == 0 ? 0u : ends[band - 1]; }
};

} // namespace sc
