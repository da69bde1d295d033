// Elementwise kernels of the projector tower that sit between its library GEMMs, fused so that each activation tensor is
// read once:
//
//   gelu_forward          h = gelu(z) = z * Phi(z), bfloat16 in and out, float32 arithmetic (the erf form, not the tanh one)
//   gelu_backward_bias    dz = dh * gelu'(z) and, in the same pass, the column sums of dz (the bias gradient of the
//                         layer before the activation), as per-row-block partial sums
//   column_sums           column sums of a bfloat16 matrix (the bias gradient of the last layer), same partials
//   fold_column_partials  adds the partials in row-block order: the bias gradients do not depend on scheduling
//
// The reference has no model; these belong to the training step this library benchmarks around its loss.
#include <stdexcept>
#include <string>

#include "api.h"
#include "common.cuh"

namespace sc {

namespace {

constexpr int tower_rows_per_block = 64;    // rows of one partial sum
constexpr int tower_columns_per_block = 256; // 32 lanes x 8 columns

// The normal distribution's cdf and pdf at z, sharing one exponential. erf comes from the five-term rational form of
// Abramowitz and Stegun 7.1.26 (absolute error below 1.5e-7, three orders of magnitude under a bfloat16's resolution)
// with one reciprocal and one base-two exponential on the special-function unit: the library erff costs about forty
// instructions per element and made these passes arithmetic-bound instead of memory-bound.
__device__ __forceinline__ void normal_cdf_pdf(float z, float& cdf, float& pdf) {
    float const x = fabsf(z) * 0.70710678118654752f;
    float const t = fast_rcp(fmaf(0.3275911f, x, 1.0f));
    float const decay = fast_ex2(-1.4426950408889634f * x * x); // exp(-z^2 / 2)
    float poly = 1.061405429f;
    poly = fmaf(poly, t, -1.453152027f);
    poly = fmaf(poly, t, 1.421413741f);
    poly = fmaf(poly, t, -0.284496736f);
    poly = fmaf(poly, t, 0.254829592f);
    float const tail = 0.5f * poly * t * decay; // (1 - erf(x)) / 2 for x >= 0
    cdf = z >= 0.0f ? 1.0f - tail : tail;
    pdf = 0.39894228040143268f * decay;
}
__device__ __forceinline__ float gelu_value(float z) {
    float cdf, pdf;
    normal_cdf_pdf(z, cdf, pdf);
    return z * cdf;
}
__device__ __forceinline__ float gelu_slope(float z) {
    float cdf, pdf;
    normal_cdf_pdf(z, cdf, pdf);
    return fmaf(z, pdf, cdf);
}
__device__ __forceinline__ void unpack8(uint4 packed, float (&v)[8]) {
    uint32_t const words[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
    for (int w = 0; w < 4; ++w) v[2 * w] = __uint_as_float(words[w] << 16), v[2 * w + 1] = __uint_as_float(words[w] & 0xFFFF0000u);
}
__device__ __forceinline__ uint4 pack8(float const (&v)[8]) {
    return make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
}

__global__ void __launch_bounds__(256) gelu_forward_kernel(uint4 const* __restrict__ z, uint4* __restrict__ h, size_t vectors) {
    // Four vectors per thread and trip, all loads issued before the first is used: the pass is bound by memory, and the
    // arithmetic of one vector would otherwise stand between consecutive loads.
    constexpr int batch = 4;
    size_t const stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; index < vectors; index += batch * stride) {
        uint4 loaded[batch];
#pragma unroll
        for (int b = 0; b < batch; ++b)
            if (index + b * stride < vectors) loaded[b] = z[index + b * stride];
#pragma unroll
        for (int b = 0; b < batch; ++b) {
            if (index + b * stride >= vectors) break;
            float v[8];
            unpack8(loaded[b], v);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = gelu_value(v[i]);
            h[index + b * stride] = pack8(v);
        }
    }
}

// One block: 64 rows x 256 columns. Thread (row group r = threadIdx.x / 32, lane) walks rows r, r + 8, ... of the block
// and keeps eight column sums; the eight row groups are then added in shared memory in a fixed order.
template <bool with_activation_>
__global__ void __launch_bounds__(256)
    column_partials_kernel(uint4 const* __restrict__ upstream, uint4 const* __restrict__ z, uint4* __restrict__ out,
                           float* __restrict__ partials, uint32_t rows, uint32_t columns) {
    __shared__ float sums[8][tower_columns_per_block];
    uint32_t const lane = threadIdx.x % 32, group = threadIdx.x / 32;
    uint32_t const column = blockIdx.x * tower_columns_per_block + lane * 8;
    uint32_t const first_row = blockIdx.y * tower_rows_per_block;
    uint32_t const vectors_per_row = columns / 8;
    float total[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (column < columns) {
        // Four rows per trip, their loads issued together; the sums still take the rows in ascending order.
        constexpr uint32_t batch = 4;
        uint32_t const end = min(first_row + tower_rows_per_block, rows);
        for (uint32_t base = first_row + group; base < end; base += 8 * batch) {
            uint4 up[batch], pre[batch];
#pragma unroll
            for (uint32_t b = 0; b < batch; ++b) {
                uint32_t const row = base + 8 * b;
                size_t const index = static_cast<size_t>(row) * vectors_per_row + column / 8;
                if (row < end && SC_IN_BOUNDS(index, static_cast<size_t>(rows) * vectors_per_row)) {
                    up[b] = upstream[index];
                    if constexpr (with_activation_) pre[b] = z[index];
                }
            }
#pragma unroll
            for (uint32_t b = 0; b < batch; ++b) {
                uint32_t const row = base + 8 * b;
                size_t const index = static_cast<size_t>(row) * vectors_per_row + column / 8;
                if (row >= end || !SC_IN_BOUNDS(index, static_cast<size_t>(rows) * vectors_per_row)) continue;
                float g[8];
                unpack8(up[b], g);
                if constexpr (with_activation_) {
                    float v[8];
                    unpack8(pre[b], v);
#pragma unroll
                    for (int i = 0; i < 8; ++i) g[i] *= gelu_slope(v[i]);
                    uint4 const rounded = pack8(g);
                    out[index] = rounded;
                    unpack8(rounded, g); // the bias gradient sums what the weight-gradient GEMM will read
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) total[i] += g[i];
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) sums[group][lane * 8 + i] = total[i];
    __syncthreads();
    uint32_t const mine = blockIdx.x * tower_columns_per_block + threadIdx.x;
    if (mine < columns) {
        float folded = 0;
#pragma unroll
        for (int g = 0; g < 8; ++g) folded += sums[g][threadIdx.x];
        partials[static_cast<size_t>(blockIdx.y) * columns + mine] = folded;
    }
}

// 32 columns x 8 row-block groups per block: thread (column, part) adds the partials of row blocks part, part + 8, ... and
// the eight parts are then added in part order, so the sum's order is fixed whatever the scheduling (and eight loads per
// column are in flight instead of one dependent chain).
__global__ void __launch_bounds__(256)
    fold_column_partials_kernel(float const* __restrict__ partials, float* __restrict__ out, uint32_t blocks, uint32_t columns,
                                void* __restrict__ out_bf16) {
    __shared__ float parts[8][32];
    uint32_t const lane = threadIdx.x % 32, part = threadIdx.x / 32;
    uint32_t const column = blockIdx.x * 32 + lane;
    float total = 0;
    if (column < columns)
        for (uint32_t block = part; block < blocks; block += 8) total += partials[static_cast<size_t>(block) * columns + column];
    parts[part][lane] = total;
    __syncthreads();
    if (part != 0 || column >= columns) return;
    float folded = 0;
#pragma unroll
    for (int other = 0; other < 8; ++other) folded += parts[other][lane];
    if (out != nullptr) out[column] = folded;
    if (out_bf16 != nullptr) static_cast<__nv_bfloat16*>(out_bf16)[column] = __float2bfloat16(folded);
}

void check_launch(char const* what) {
    cudaError_t const error = cudaGetLastError();
    if (error != cudaSuccess) throw std::runtime_error(std::string(what) + " launch failed: " + cudaGetErrorString(error));
    note_launch();
}

void check_matrix(uint32_t rows, uint32_t columns, char const* what) {
    if (rows == 0 || columns == 0 || columns % 8) throw std::runtime_error(std::string(what) + ": columns must be a positive multiple of 8");
}

} // namespace

uint32_t tower_partial_blocks(uint32_t rows) { return (rows + tower_rows_per_block - 1) / tower_rows_per_block; }

void launch_gelu_forward(void const* z_bf16, void* h_bf16, size_t scalars, int multiprocessors, cudaStream_t stream) {
    if (scalars % 8) throw std::runtime_error("gelu_forward: the element count must be a multiple of 8");
    size_t const vectors = scalars / 8;
    size_t blocks = (vectors + 255) / 256;
    size_t const cap = static_cast<size_t>(multiprocessors > 0 ? multiprocessors : 148) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) return;
    gelu_forward_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<uint4 const*>(z_bf16), static_cast<uint4*>(h_bf16), vectors);
    check_launch("gelu_forward");
}

void launch_gelu_backward_bias(void const* upstream_bf16, void const* z_bf16, void* dz_bf16, float* partials, void* bias_grad_bf16,
                               uint32_t rows, uint32_t columns, cudaStream_t stream) {
    check_matrix(rows, columns, "gelu_backward_bias");
    dim3 const grid((columns + tower_columns_per_block - 1) / tower_columns_per_block, tower_partial_blocks(rows));
    column_partials_kernel<true><<<grid, 256, 0, stream>>>(static_cast<uint4 const*>(upstream_bf16), static_cast<uint4 const*>(z_bf16),
                                                            static_cast<uint4*>(dz_bf16), partials, rows, columns);
    check_launch("gelu_backward_bias");
    fold_column_partials_kernel<<<(columns + 31) / 32, 256, 0, stream>>>(partials, nullptr, grid.y, columns, bias_grad_bf16);
    check_launch("fold_column_partials");
}

void launch_column_sums(void const* matrix_bf16, float* partials, void* sums_bf16, uint32_t rows, uint32_t columns,
                        cudaStream_t stream) {
    check_matrix(rows, columns, "column_sums");
    dim3 const grid((columns + tower_columns_per_block - 1) / tower_columns_per_block, tower_partial_blocks(rows));
    column_partials_kernel<false><<<grid, 256, 0, stream>>>(static_cast<uint4 const*>(matrix_bf16), nullptr, nullptr, partials, rows, columns);
    check_launch("column_sums");
    fold_column_partials_kernel<<<(columns + 31) / 32, 256, 0, stream>>>(partials, nullptr, grid.y, columns, sums_bf16);
    check_launch("fold_column_partials");
}

SC_DEFINE_BOUNDS_READER(bounds_record_tower)

} // namespace sc
