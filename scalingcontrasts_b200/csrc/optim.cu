// AdamW with decoupled weight decay over a short list of tensors in one launch: the optimizer step of the training
// benchmark. Parameters and gradients are bfloat16 or float32; both moments are kept in float32 whatever the parameter's
// type (a bfloat16 second moment cannot follow gradients whose squares differ by more than its eight bits). Every element
// is read and written once: 2 + 2 + 4 + 4 bytes in, 2 + 4 + 4 out per bfloat16 parameter.
//
//   p <- p * (1 - lr * decay);  m <- b1 * m + (1 - b1) * g;  v <- b2 * v + (1 - b2) * g * g
//   p <- p - (lr / (1 - b1^t)) * m / (sqrt(v) / sqrt(1 - b2^t) + eps)
//
// The bias corrections are computed on the host from the step count and arrive as two floats. A block owns 2048
// consecutive elements of one tensor; which tensor is found by walking the launch's table of first blocks (at most eight
// entries, in the kernel's parameters).
//
// The reference has no optimizer (it benchmarks a loss step only, scalingcontrasts.cu:294-311).
#include <cmath>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "api.h"
#include "common.cuh"

namespace sc {

namespace {

constexpr uint32_t adamw_block_elements = 2048; // 256 threads x 8

struct adamw_table {
    adamw_tensor tensors[adamw_max_tensors];
    uint32_t first_block[adamw_max_tensors + 1];
    uint32_t used;
};

struct adamw_constants {
    float keep;        // 1 - lr * decay
    float b1, b2;      // the moments' decay rates
    float step_size;   // lr / (1 - b1^t)
    float inverse_root_correction2; // 1 / sqrt(1 - b2^t)
    float eps;
};

__device__ __forceinline__ float adamw_update(float p, float g, float& m, float& v, adamw_constants const& c) {
    m = fmaf(c.b1, m, (1.0f - c.b1) * g);
    v = fmaf(c.b2, v, (1.0f - c.b2) * g * g);
    float const denominator = fmaf(sqrtf(v), c.inverse_root_correction2, c.eps);
    return fmaf(-c.step_size, __fdividef(m, denominator), p * c.keep);
}

__global__ void __launch_bounds__(256) adamw_kernel(const adamw_table table, const adamw_constants c) {
    uint32_t index = 0;
    while (index + 1 < table.used && blockIdx.x >= table.first_block[index + 1]) ++index;
    adamw_tensor const t = table.tensors[index];
    size_t const begin = static_cast<size_t>(blockIdx.x - table.first_block[index]) * adamw_block_elements;
    if (t.is_bf16 && t.vectorised) {
        size_t const at = begin + threadIdx.x * 8u;
        if (at >= t.count || !SC_IN_BOUNDS(at + 7, t.count)) return;
        uint4 const packed_p = *reinterpret_cast<uint4 const*>(static_cast<__nv_bfloat16 const*>(t.param) + at);
        uint4 const packed_g = *reinterpret_cast<uint4 const*>(static_cast<__nv_bfloat16 const*>(t.grad) + at);
        float4 m_lo = *reinterpret_cast<float4 const*>(t.exp_avg + at), m_hi = *reinterpret_cast<float4 const*>(t.exp_avg + at + 4);
        float4 v_lo = *reinterpret_cast<float4 const*>(t.exp_avg_sq + at), v_hi = *reinterpret_cast<float4 const*>(t.exp_avg_sq + at + 4);
        uint32_t const words_p[4] = {packed_p.x, packed_p.y, packed_p.z, packed_p.w};
        uint32_t const words_g[4] = {packed_g.x, packed_g.y, packed_g.z, packed_g.w};
        float m[8] = {m_lo.x, m_lo.y, m_lo.z, m_lo.w, m_hi.x, m_hi.y, m_hi.z, m_hi.w};
        float v[8] = {v_lo.x, v_lo.y, v_lo.z, v_lo.w, v_hi.x, v_hi.y, v_hi.z, v_hi.w};
        float p[8];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            p[2 * w] = adamw_update(__uint_as_float(words_p[w] << 16), __uint_as_float(words_g[w] << 16), m[2 * w], v[2 * w], c);
            p[2 * w + 1] = adamw_update(__uint_as_float(words_p[w] & 0xFFFF0000u), __uint_as_float(words_g[w] & 0xFFFF0000u),
                                        m[2 * w + 1], v[2 * w + 1], c);
        }
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(t.param) + at) =
            make_uint4(pack_bf16x2(p[0], p[1]), pack_bf16x2(p[2], p[3]), pack_bf16x2(p[4], p[5]), pack_bf16x2(p[6], p[7]));
        *reinterpret_cast<float4*>(t.exp_avg + at) = make_float4(m[0], m[1], m[2], m[3]);
        *reinterpret_cast<float4*>(t.exp_avg + at + 4) = make_float4(m[4], m[5], m[6], m[7]);
        *reinterpret_cast<float4*>(t.exp_avg_sq + at) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(t.exp_avg_sq + at + 4) = make_float4(v[4], v[5], v[6], v[7]);
        return;
    }
    // any count, any alignment, either type: one element per thread and trip
    for (size_t at = begin + threadIdx.x; at < begin + adamw_block_elements && at < t.count; at += blockDim.x) {
        if (!SC_IN_BOUNDS(at, t.count)) break;
        float m = t.exp_avg[at], v = t.exp_avg_sq[at];
        if (t.is_bf16) {
            __nv_bfloat16* const param = static_cast<__nv_bfloat16*>(t.param);
            float const updated = adamw_update(__bfloat162float(param[at]),
                                               __bfloat162float(static_cast<__nv_bfloat16 const*>(t.grad)[at]), m, v, c);
            param[at] = __float2bfloat16(updated);
        } else {
            float* const param = static_cast<float*>(t.param);
            param[at] = adamw_update(param[at], static_cast<float const*>(t.grad)[at], m, v, c);
        }
        t.exp_avg[at] = m, t.exp_avg_sq[at] = v;
    }
}

} // namespace

void launch_adamw(adamw_tensor const* tensors, uint32_t count, float lr, float beta1, float beta2, float eps, float decay,
                  uint64_t step, cudaStream_t stream) {
    if (step < 1) throw std::runtime_error("adamw: the step count starts at 1");
    if (!(beta1 >= 0.0f && beta1 < 1.0f && beta2 >= 0.0f && beta2 < 1.0f)) throw std::runtime_error("adamw: betas must lie in [0, 1)");
    for (uint32_t i = 0; i < count; ++i) {
        adamw_tensor const& t = tensors[i];
        if (!t.param || !t.grad || !t.exp_avg || !t.exp_avg_sq) throw std::runtime_error("adamw: a null pointer among the tensors");
        if (t.count == 0) throw std::runtime_error("adamw: an empty tensor");
        if (t.count > (1ull << 40)) throw std::runtime_error("adamw: tensor too large for one launch's block count");
    }
    double const correction1 = 1.0 - std::pow(static_cast<double>(beta1), static_cast<double>(step));
    double const correction2 = 1.0 - std::pow(static_cast<double>(beta2), static_cast<double>(step));
    adamw_constants c{};
    c.keep = 1.0f - lr * decay, c.b1 = beta1, c.b2 = beta2, c.eps = eps;
    c.step_size = static_cast<float>(lr / correction1);
    c.inverse_root_correction2 = static_cast<float>(1.0 / std::sqrt(correction2));
    for (uint32_t first = 0; first < count; first += adamw_max_tensors) {
        adamw_table table{};
        uint32_t blocks = 0;
        for (uint32_t i = first; i < count && table.used < adamw_max_tensors; ++i) {
            adamw_tensor t = tensors[i];
            auto const aligned = [](void const* pointer) { return reinterpret_cast<uintptr_t>(pointer) % 16 == 0; };
            t.vectorised = t.is_bf16 && t.count % 8 == 0 && aligned(t.param) && aligned(t.grad) && aligned(t.exp_avg) &&
                                   aligned(t.exp_avg_sq)
                               ? 1u
                               : 0u;
            table.tensors[table.used] = t;
            table.first_block[table.used] = blocks;
            blocks += static_cast<uint32_t>((t.count + adamw_block_elements - 1) / adamw_block_elements);
            ++table.used;
        }
        table.first_block[table.used] = blocks;
        adamw_kernel<<<blocks, 256, 0, stream>>>(table, c);
        cudaError_t const error = cudaGetLastError();
        if (error != cudaSuccess) throw std::runtime_error(std::string("adamw launch failed: ") + cudaGetErrorString(error));
        note_launch();
    }
}

SC_DEFINE_BOUNDS_READER(bounds_record_optim)

} // namespace sc
