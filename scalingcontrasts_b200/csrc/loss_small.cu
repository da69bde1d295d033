// The memory-bound kernels around the two tile kernels of the streamed loss, and the keyed generators / validators.
//
//   prefix_norms      per row, the inverse norm of every prefix (and optionally a copy of the row into symmetric
//                     memory, so that publishing a block to the peers costs no extra pass), then per 64 rows the
//                     largest inverse norm, which lets a tile prove that no cosine of it sits on the floor
//   transpose         [R, H] -> [H, R] so that the gradient tiles read candidates K-major
//   pull              peer block -> local staging by plain 16-byte loads and stores
//   fold_partials     per row, adds the forward kernel's per-run partials in run order (deterministic)
//   finalize          folds the L2-normalisation's self term into the query gradient and casts to bfloat16
//   sum_summands      fixed-tree sums of the row accumulators into the loss summands
//
// Parity: transpose_cuda_, prefix_inverse_norms_cuda_, fold_partials_cuda_, finalize_cuda_, sum_summands_cuda_
// (scalingcontrasts.cuh:660-686, 1138-1177); keyed_* and count_* (scalingcontrasts.cu:48-105). The staging pull
// replaces the reference's cudaMemcpyAsync (scalingcontrasts.cuh:1262-1265).
#include <stdexcept>
#include <string>

#include "api.h"
#include "common.cuh"

namespace sc {

namespace {

void check_launch(char const* what) {
    cudaError_t const error = cudaGetLastError();
    if (error != cudaSuccess) throw std::runtime_error(std::string(what) + " launch failed: " + cudaGetErrorString(error));
    note_launch();
}

ladder_t to_device(ladder_host const& host) {
    ladder_t ladder{};
    ladder.count = host.count;
    for (int i = 0; i < 8; ++i) ladder.ends[i] = host.ends[i];
    return ladder;
}

// One warp per row. Each lane reads 16-byte vectors (8 channels); band edges are multiples of 16 channels, so a vector
// never straddles two bands.
__global__ void __launch_bounds__(256)
    prefix_norms_kernel(uint4 const* __restrict__ rows, uint4* __restrict__ copy, float* __restrict__ inverse_norms,
                        uint32_t row_count, uint32_t hidden, ladder_t ladder) {
    uint32_t const warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    uint32_t const row = blockIdx.x * 8 + warp;
    if (row >= row_count) return;
    uint32_t const vectors = hidden / 8;
    float sums[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (uint32_t v = lane; v < vectors; v += 32) {
        if (!SC_IN_BOUNDS(static_cast<size_t>(row) * vectors + v, static_cast<size_t>(row_count) * vectors)) continue;
        uint4 const packed = rows[static_cast<size_t>(row) * vectors + v];
        if (copy != nullptr) copy[static_cast<size_t>(row) * vectors + v] = packed;
        uint32_t const words[4] = {packed.x, packed.y, packed.z, packed.w};
        float square = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            float const lo = __uint_as_float(words[w] << 16), hi = __uint_as_float(words[w] & 0xFFFF0000u);
            square = fmaf(lo, lo, square);
            square = fmaf(hi, hi, square);
        }
        uint32_t const channel = v * 8;
#pragma unroll
        for (int band = 0; band < 8; ++band)
            if (band < ladder.count && channel >= ladder.begin(band) && channel < ladder.ends[band]) sums[band] += square;
    }
    float running = 0;
#pragma unroll
    for (int band = 0; band < 8; ++band) {
        if (band >= ladder.count) break;
        float total = sums[band];
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) total += __shfl_xor_sync(0xFFFFFFFFu, total, offset);
        running += total;
        if (lane == 0 && SC_IN_BOUNDS(static_cast<size_t>(band) * row_count + row, static_cast<size_t>(ladder.count) * row_count))
            inverse_norms[static_cast<size_t>(band) * row_count + row] = running > 0.0f ? rsqrtf(running) : 0.0f;
    }
}

// tile_max[band, t] = max over rows [64 t, 64 t + 64) of inverse_norms[band, row].
__global__ void tile_max_kernel(float const* __restrict__ inverse_norms, float* __restrict__ tile_max, uint32_t row_count,
                                uint32_t bands) {
    uint32_t const tiles = row_count / 64;
    uint32_t const index = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    uint32_t const lane = threadIdx.x % 32;
    if (index >= tiles * bands) return;
    uint32_t const band = index / tiles, tile = index % tiles;
    float const* base = inverse_norms + static_cast<size_t>(band) * row_count + tile * 64;
    if (!SC_IN_BOUNDS(static_cast<size_t>(band) * row_count + tile * 64 + lane + 32, static_cast<size_t>(bands) * row_count)) return;
    float value = fmaxf(base[lane], base[lane + 32]);
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) value = fmaxf(value, __shfl_xor_sync(0xFFFFFFFFu, value, offset));
    if (lane == 0) tile_max[static_cast<size_t>(band) * tiles + tile] = value;
}

__global__ void __launch_bounds__(256)
    transpose_kernel(__nv_bfloat16 const* __restrict__ in, __nv_bfloat16* __restrict__ out, uint32_t rows, uint32_t hidden) {
    __shared__ __nv_bfloat16 tile[32][33];
    uint32_t const column = blockIdx.x * 32 + threadIdx.x;
    for (uint32_t r = threadIdx.y; r < 32; r += 8) {
        uint32_t const row = blockIdx.y * 32 + r;
        if (row < rows && column < hidden && SC_IN_BOUNDS(static_cast<size_t>(row) * hidden + column, static_cast<size_t>(rows) * hidden))
            tile[r][threadIdx.x] = in[static_cast<size_t>(row) * hidden + column];
    }
    __syncthreads();
    uint32_t const out_column = blockIdx.y * 32 + threadIdx.x;
    for (uint32_t r = threadIdx.y; r < 32; r += 8) {
        uint32_t const out_row = blockIdx.x * 32 + r;
        if (out_row < hidden && out_column < rows &&
            SC_IN_BOUNDS(static_cast<size_t>(out_row) * rows + out_column, static_cast<size_t>(rows) * hidden))
            out[static_cast<size_t>(out_row) * rows + out_column] = tile[threadIdx.x][r];
    }
}

__device__ __forceinline__ void copy_vectors(uint4 const* src, uint4* dst, size_t vectors, size_t thread, size_t threads) {
    size_t index = thread;
    for (; index + 3 * threads < vectors; index += 4 * threads) {
        uint4 a = src[index], b = src[index + threads], c = src[index + 2 * threads], d = src[index + 3 * threads];
        dst[index] = a, dst[index + threads] = b, dst[index + 2 * threads] = c, dst[index + 3 * threads] = d;
    }
    for (; index < vectors; index += threads) dst[index] = src[index];
}

__global__ void __launch_bounds__(256) pull_kernel(pull_request request) {
    size_t const thread = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    size_t const threads = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (int part = 0; part < 2; ++part)
        if (request.bytes[part] != 0)
            copy_vectors(static_cast<uint4 const*>(request.src[part]), static_cast<uint4*>(request.dst[part]),
                         request.bytes[part] / 16, thread, threads);
}

__global__ void __launch_bounds__(256)
    fold_partials_kernel(float const* __restrict__ partials, float* __restrict__ accumulators, uint32_t rows, uint32_t slots,
                         uint32_t quantities) {
    uint32_t const row = blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t const quantity = blockIdx.y;
    if (row >= rows) return;
    float total = 0;
#pragma unroll 8
    for (uint32_t slot = 0; slot < slots; ++slot)
        if (SC_IN_BOUNDS((static_cast<size_t>(slot) * quantities + quantity) * rows + row, static_cast<size_t>(slots) * quantities * rows))
            total += partials[(static_cast<size_t>(slot) * quantities + quantity) * rows + row];
    accumulators[static_cast<size_t>(quantity) * rows + row] += total;
}

// Row accumulators are laid out [quantity, row] with quantities: 0 bias grad, 1 log-beta grad, 2..2+K prefix losses,
// 2+K..2+2K self coefficients.
__global__ void __launch_bounds__(128)
    finalize_kernel(uint4 const* __restrict__ queries, float const* __restrict__ inverse_norms,
                    float const* __restrict__ accumulators, float const* __restrict__ query_gradient,
                    uint4* __restrict__ gradient_out, uint32_t rows, uint32_t hidden, ladder_t ladder) {
    uint32_t const row = blockIdx.x;
    __shared__ float fold_from[8]; // fold_from[b] = sum over bands k >= b of coefficient_k * inverse_norm_k^2
    if (threadIdx.x == 0) {
        float running = 0;
        for (int band = static_cast<int>(ladder.count) - 1; band >= 0; --band) {
            float const inverse = inverse_norms[static_cast<size_t>(band) * rows + row];
            float const coefficient = accumulators[static_cast<size_t>(2 + ladder.count + band) * rows + row];
            running += coefficient * inverse * inverse;
            fold_from[band] = running;
        }
    }
    __syncthreads();
    uint32_t const vectors = hidden / 8;
    for (uint32_t v = threadIdx.x; v < vectors; v += blockDim.x) {
        uint32_t const channel = v * 8;
        uint32_t band = 0;
        while (band + 1 < ladder.count && channel >= ladder.ends[band]) ++band;
        float const fold = fold_from[band];
        if (!SC_IN_BOUNDS(static_cast<size_t>(row) * hidden + channel + 7, static_cast<size_t>(rows) * hidden)) continue;
        uint4 const packed = queries[static_cast<size_t>(row) * vectors + v];
        float4 const g0 = *reinterpret_cast<float4 const*>(query_gradient + static_cast<size_t>(row) * hidden + channel);
        float4 const g1 = *reinterpret_cast<float4 const*>(query_gradient + static_cast<size_t>(row) * hidden + channel + 4);
        uint32_t const words[4] = {packed.x, packed.y, packed.z, packed.w};
        float const g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        uint32_t out[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            float const lo = __uint_as_float(words[w] << 16), hi = __uint_as_float(words[w] & 0xFFFF0000u);
            out[w] = pack_bf16x2(fmaf(-fold, lo, g[2 * w]), fmaf(-fold, hi, g[2 * w + 1]));
        }
        gradient_out[static_cast<size_t>(row) * vectors + v] = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

// One block; a fixed reduction tree, so the bits do not depend on anything but the inputs.
__global__ void __launch_bounds__(1024)
    sum_summands_kernel(float const* __restrict__ accumulators, float* __restrict__ summands, uint32_t rows, uint32_t prefixes) {
    __shared__ float scratch[32];
    __shared__ float totals[10];
    uint32_t const quantities = 2 + prefixes;
    for (uint32_t quantity = 0; quantity < quantities; ++quantity) {
        // Four 16-byte loads in flight per thread before anything is added (rows are a multiple of 128, so a quantity's
        // rows are whole, aligned vectors): one round trip to memory per quantity instead of one per row a thread owns.
        float partial = 0;
        float4 const* const vectors = reinterpret_cast<float4 const*>(accumulators + static_cast<size_t>(quantity) * rows);
        uint32_t const count = rows / 4;
        for (uint32_t first = threadIdx.x; first < count; first += 4 * blockDim.x) {
            float4 held[4];
#pragma unroll
            for (uint32_t u = 0; u < 4; ++u) {
                uint32_t const index = first + u * blockDim.x;
                held[u] = index < count ? vectors[index] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (uint32_t u = 0; u < 4; ++u) partial += (held[u].x + held[u].y) + (held[u].z + held[u].w);
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) partial += __shfl_xor_sync(0xFFFFFFFFu, partial, offset);
        if (threadIdx.x % 32 == 0) scratch[threadIdx.x / 32] = partial;
        __syncthreads();
        if (threadIdx.x < 32) {
            float value = threadIdx.x < blockDim.x / 32 ? scratch[threadIdx.x] : 0.0f;
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_xor_sync(0xFFFFFFFFu, value, offset);
            if (threadIdx.x == 0) totals[quantity] = value;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        float loss = 0;
        for (uint32_t band = 0; band < prefixes; ++band) loss += totals[2 + band];
        summands[0] = loss;
        summands[1] = totals[0];
        summands[2] = totals[1];
        summands[3] = 0.0f;
        for (uint32_t band = 0; band < 8; ++band) summands[4 + band] = band < prefixes ? totals[2 + band] : 0.0f;
    }
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t value) {
    value = (value ^ (value >> 30)) * 0xBF58476D1CE4E5B9ull;
    value = (value ^ (value >> 27)) * 0x94D049BB133111EBull;
    return value ^ (value >> 31);
}

__global__ void keyed_embeddings_kernel(__nv_bfloat16* rows, uint32_t row_count, uint32_t hidden, uint64_t salt, float scale) {
    uint64_t const row = blockIdx.x;
    for (uint32_t channel = threadIdx.x; channel < hidden; channel += blockDim.x) {
        uint64_t const bits = splitmix64((salt * row_count + row) * hidden + channel);
        rows[row * hidden + channel] = __float2bfloat16((static_cast<float>(bits >> 40) * 0x1.0p-24f - 0.5f) * scale);
    }
}

__global__ void keyed_integers_kernel(float* out, size_t scalars, size_t first, uint32_t members, uint32_t member) {
    size_t const index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= scalars) return;
    out[index] = static_cast<float>(splitmix64((first + index) * members + member) >> 52);
}

__global__ void keyed_fractions_kernel(float* out, size_t scalars, size_t first, uint32_t members, uint32_t member) {
    size_t const index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= scalars) return;
    out[index] = static_cast<float>(splitmix64((first + index) * members + member) >> 40) * 0x1.0p-24f - 0.5f;
}

__global__ void count_wrong_sums_kernel(float const* values, size_t scalars, size_t first, uint32_t members,
                                        unsigned long long* counter) {
    size_t const index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= scalars) return;
    float expected = 0;
    for (uint32_t member = 0; member < members; ++member)
        expected += static_cast<float>(splitmix64((first + index) * members + member) >> 52);
    if (values[index] != expected) atomicAdd(counter, 1ull);
}

__global__ void count_differences_kernel(uint32_t const* values, uint32_t const* expected, size_t scalars,
                                         unsigned long long* counter) {
    size_t const index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= scalars) return;
    if (values[index] != expected[index]) atomicAdd(counter, 1ull);
}

__global__ void scale_cast_kernel(float const* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t scalars, float scale) {
    size_t const index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index < scalars) dst[index] = __float2bfloat16(src[index] * scale);
}

int blocks_of(size_t items, int per_block) { return static_cast<int>((items + per_block - 1) / per_block); }

} // namespace

bool bounds_build() { return SC_BOUNDS != 0; }
SC_DEFINE_BOUNDS_READER(bounds_record_small)

void launch_prefix_norms(void const* rows_bf16, void* copy_bf16, float* inverse_norms, float* tile_max, uint32_t rows,
                         uint32_t hidden, ladder_host const& ladder, cudaStream_t stream) {
    if (hidden % 8) throw std::runtime_error("prefix_norms: hidden must be a multiple of 8");
    prefix_norms_kernel<<<blocks_of(rows, 8), 256, 0, stream>>>(static_cast<uint4 const*>(rows_bf16),
                                                               static_cast<uint4*>(copy_bf16), inverse_norms, rows, hidden,
                                                               to_device(ladder));
    check_launch("prefix_norms");
    if (tile_max != nullptr) {
        if (rows % 64) throw std::runtime_error("prefix_norms: rows must be a multiple of 64 for tile maxima");
        uint32_t const items = rows / 64 * ladder.count;
        tile_max_kernel<<<blocks_of(items, 8), 256, 0, stream>>>(inverse_norms, tile_max, rows, ladder.count);
        check_launch("tile_max");
    }
}

void launch_transpose(void const* rows_bf16, void* transposed_bf16, uint32_t rows, uint32_t hidden, cudaStream_t stream) {
    dim3 const grid((hidden + 31) / 32, (rows + 31) / 32), block(32, 8);
    transpose_kernel<<<grid, block, 0, stream>>>(static_cast<__nv_bfloat16 const*>(rows_bf16),
                                                 static_cast<__nv_bfloat16*>(transposed_bf16), rows, hidden);
    check_launch("transpose");
}

void launch_pull(void const* src0, void* dst0, size_t bytes0, void const* src1, void* dst1, size_t bytes1, int blocks,
                 cudaStream_t stream) {
    if (bytes0 % 16 || bytes1 % 16) throw std::runtime_error("pull: sizes must be multiples of 16 bytes");
    pull_request request{};
    request.src[0] = src0, request.dst[0] = dst0, request.bytes[0] = bytes0;
    request.src[1] = src1, request.dst[1] = dst1, request.bytes[1] = bytes1;
    pull_kernel<<<blocks < 1 ? 1 : blocks, 256, 0, stream>>>(request);
    check_launch("pull");
}

void launch_fold_partials(float const* partials, float* row_accumulators, uint32_t rows, uint32_t slots,
                          uint32_t quantities, cudaStream_t stream) {
    fold_partials_kernel<<<dim3(blocks_of(rows, 256), quantities), 256, 0, stream>>>(partials, row_accumulators, rows, slots,
                                                                                   quantities);
    check_launch("fold_partials");
}

void launch_finalize(void const* queries_bf16, float const* inverse_norms, float const* row_accumulators,
                     float const* query_gradient, void* gradient_out_bf16, uint32_t rows, uint32_t hidden,
                     ladder_host const& ladder, cudaStream_t stream) {
    finalize_kernel<<<rows, 128, 0, stream>>>(static_cast<uint4 const*>(queries_bf16), inverse_norms, row_accumulators,
                                              query_gradient, static_cast<uint4*>(gradient_out_bf16), rows, hidden,
                                              to_device(ladder));
    check_launch("finalize");
}

void launch_sum_summands(float const* row_accumulators, float* summands, uint32_t rows, uint32_t prefixes,
                         cudaStream_t stream) {
    if (rows % 4 || reinterpret_cast<uintptr_t>(row_accumulators) % 16)
        throw std::runtime_error("sum_summands: rows must be a multiple of 4 and the accumulators 16-byte aligned");
    sum_summands_kernel<<<1, 1024, 0, stream>>>(row_accumulators, summands, rows, prefixes);
    check_launch("sum_summands");
}

void launch_keyed_embeddings(void* rows_bf16, uint32_t rows, uint32_t hidden, uint64_t salt, float scale,
                             cudaStream_t stream) {
    keyed_embeddings_kernel<<<rows, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(rows_bf16), rows, hidden, salt, scale);
    check_launch("keyed_embeddings");
}

void launch_keyed_integers(float* out, size_t scalars, size_t first, uint32_t members, uint32_t member,
                           cudaStream_t stream) {
    keyed_integers_kernel<<<blocks_of(scalars, 256), 256, 0, stream>>>(out, scalars, first, members, member);
    check_launch("keyed_integers");
}

void launch_keyed_fractions(float* out, size_t scalars, size_t first, uint32_t members, uint32_t member,
                            cudaStream_t stream) {
    keyed_fractions_kernel<<<blocks_of(scalars, 256), 256, 0, stream>>>(out, scalars, first, members, member);
    check_launch("keyed_fractions");
}

void launch_count_wrong_sums(float const* values, size_t scalars, size_t first, uint32_t members,
                             unsigned long long* counter, cudaStream_t stream) {
    count_wrong_sums_kernel<<<blocks_of(scalars, 256), 256, 0, stream>>>(values, scalars, first, members, counter);
    check_launch("count_wrong_sums");
}

void launch_count_differences(float const* values, float const* expected, size_t scalars, unsigned long long* counter,
                              cudaStream_t stream) {
    count_differences_kernel<<<blocks_of(scalars, 256), 256, 0, stream>>>(reinterpret_cast<uint32_t const*>(values),
                                                                       reinterpret_cast<uint32_t const*>(expected), scalars,
                                                                       counter);
    check_launch("count_differences");
}

void launch_scale_cast(float const* src, void* dst_bf16, size_t scalars, float scale, cudaStream_t stream) {
    scale_cast_kernel<<<blocks_of(scalars, 256), 256, 0, stream>>>(src, static_cast<__nv_bfloat16*>(dst_bf16), scalars, scale);
    check_launch("scale_cast");
}

} // namespace sc
