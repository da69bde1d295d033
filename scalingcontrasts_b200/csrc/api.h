// Host-side entry points of the native layer. Plain C++ types only, so that the kernel translation units need no
// framework headers; bindings.cpp wraps these for Python.
//
// Every launcher enqueues on the given stream and returns without synchronising. Errors that the host can see at
// launch time throw std::runtime_error; errors that only the device can see (a wait that ran out) land in the status
// block passed to the kernel.
#pragma once

#include <array>
#include <vector>
#include <cstddef>
#include <cstdint>
#include <string>

#include <cuda_runtime.h>

namespace sc {

constexpr int max_prefixes = 8;

struct ladder_host {
    uint32_t count;
    uint32_t ends[max_prefixes];
};

// Number of kernels of this library launched so far by this process (for the bench's launch accounting).
uint64_t launch_count();
void note_launch(uint64_t launches = 1);

// -------- collectives (collectives.cu) ---------------------------------------------------------------------------
// The control block of one member: its own replica's counters, and how to reach everyone's arrival flag.
struct control_view {
    uint32_t* multicast_flag;        // multicast alias of the arrival flag; null in a peer (non-multicast) domain
    uint32_t* own_flag;              // this member's copy of the arrival flag
    uint32_t* own_round;             // arrivals this member has consumed
    uint32_t* own_finished;          // blocks of the running kernel that are done
    uint32_t* status;                // status block (status_words words)
    uint32_t* peer_flags[16];        // every member's arrival flag as seen from this GPU (peer domain)
    uint32_t members;
    uint32_t member;
    uint64_t budget_ns;
};

enum class payload_type : int { f32 = 0, bf16 = 1 };

void launch_barrier(control_view const& control, cudaStream_t stream);
// In place over `scalars` elements starting at element offset `first` of the payload. `multicast` is the multicast
// alias of the payload (null in a peer domain, where `replicas` lists every member's copy). `scale` multiplies the
// reduced value before it is stored.
void launch_all_reduce(control_view const& control, void* multicast, void* const* replicas, size_t first,
                       size_t scalars, payload_type type, float scale, int multiprocessors, cudaStream_t stream);
// The latency form for payloads of at most one staging slot: one arrival round instead of two. `own_payload` is this
// member's copy of the payload (summed in place, every member computing identical bits); the staging area holds two sets
// of `members` slots of `slot_bytes` each and is given as its multicast alias (null in a peer domain), every member's
// copy (peer domain) and this member's copy.
void launch_all_reduce_small(control_view const& control, void* own_payload, void* multicast_slots, void* const* slot_replicas,
                             void* own_slots, size_t scalars, payload_type type, float scale, size_t slot_bytes,
                             cudaStream_t stream);
// 1 when the last collective launched by this process went through the multicast alias (multimem instructions), 0 when
// it used peer loads and stores, -1 before the first.
int last_collective_path();
// Member m ends with the reduced elements [first + m*shard, first + (m+1)*shard) in its own replica. When
// `out_f32` is not null the shard goes there instead (as float32, scaled), leaving the payload untouched.
void launch_reduce_scatter(control_view const& control, void* multicast, void* const* replicas, void* own, size_t first,
                           size_t shard_scalars, payload_type type, float scale, float* out_f32, int multiprocessors,
                           cudaStream_t stream);
// Makes a wait of this member run out on purpose: consumes one round that nobody arrives for. Host-driven test hook
// for the timeout path; uses a flag that nothing sets, never a fault.
void launch_expect_arrivals(control_view const& control, uint32_t arrivals, cudaStream_t stream);
void preload_collective_kernels();

// -------- small loss kernels (loss_small.cu) ---------------------------------------------------------------------
void launch_prefix_norms(void const* rows_bf16, void* copy_bf16, float* inverse_norms, float* tile_max, uint32_t rows,
                         uint32_t hidden, ladder_host const& ladder, cudaStream_t stream);
void launch_transpose(void const* rows_bf16, void* transposed_bf16, uint32_t rows, uint32_t hidden, cudaStream_t stream);
void launch_pull(void const* src0, void* dst0, size_t bytes0, void const* src1, void* dst1, size_t bytes1, int blocks,
                 cudaStream_t stream);
void launch_fold_partials(float const* partials, float* row_accumulators, uint32_t rows, uint32_t slots,
                          uint32_t quantities, cudaStream_t stream);
void launch_finalize(void const* queries_bf16, float const* inverse_norms, float const* row_accumulators,
                     float const* query_gradient, void* gradient_out_bf16, uint32_t rows, uint32_t hidden,
                     ladder_host const& ladder, cudaStream_t stream);
void launch_sum_summands(float const* row_accumulators, float* summands, uint32_t rows, uint32_t prefixes,
                         cudaStream_t stream);
void launch_keyed_embeddings(void* rows_bf16, uint32_t rows, uint32_t hidden, uint64_t salt, float scale,
                             cudaStream_t stream);
void launch_keyed_integers(float* out, size_t scalars, size_t first, uint32_t members, uint32_t member,
                           cudaStream_t stream);
void launch_keyed_fractions(float* out, size_t scalars, size_t first, uint32_t members, uint32_t member,
                            cudaStream_t stream);
void launch_count_wrong_sums(float const* values, size_t scalars, size_t first, uint32_t members,
                             unsigned long long* counter, cudaStream_t stream);
void launch_count_differences(float const* values, float const* expected, size_t scalars, unsigned long long* counter,
                              cudaStream_t stream);
void launch_scale_cast(float const* src, void* dst_bf16, size_t scalars, float scale, cudaStream_t stream);

// -------- tile kernels (loss_fwd.cu, loss_bwd.cu) ----------------------------------------------------------------
struct pull_request {
    void const* src[2];
    void* dst[2];
    size_t bytes[2]; // multiples of 16
};

struct forward_arguments {
    void const* queries_bf16;        // [rows_q, hidden], local memory
    void const* candidates_bf16;     // [rows_c, hidden], local memory (a staged copy when the block is a peer's)
    float const* query_inverse_norms;     // [K, rows_q]
    float const* candidate_inverse_norms; // [K, rows_c]
    float const* candidate_tile_max;      // [K, rows_c / 64]
    void* gradient_cube_bf16;        // [K, rows_q, rows_c], WITHOUT the factor 2 / live (the backward launch applies it)
    float* partials;                 // [slots, quantities, rows_q]
    uint32_t* status;
    uint32_t rows_q, rows_c, hidden;
    ladder_host ladder;
    uint32_t tiles_per_run;
    float beta, bias, weight;
    float const* scalars;            // optional device {beta, bias}; overrides the two floats above when set
    uint64_t query_base, candidate_base;
    uint32_t spec_code;
    uint64_t budget_ns;
    pull_request pull;               // optional: bytes == 0 means nothing to pull
    // Optional phase timers, live only in a build with -DSC_FWD_TRACE=1 and ignored otherwise (device array of
    // forward_trace_slots counters, zeroed by the caller): CTA 0 adds the cycles
    // it spends in 0 producer issue, 1 producer waiting for a free stage, 2 UMMA issue, 3 UMMA waiting for a stage,
    // 4 UMMA waiting for a slot, 5 epilogue between tiles, 6 epilogue waiting for a tile, 7 cell pass, 8 suffix pass.
    unsigned long long* trace;
    int multiprocessors;
    // The fused form: the same launch also folds the gradient patches into `query_gradient` (tensor-core GEMM beside
    // the scoring), so no gradient cube exists. `gradient_cube_bf16` is then unused; the patches of a work item pass
    // through `fused_scratch_bf16` (forward_fused_scratch_bytes() bytes, contents meaningless between launches).
    bool fused;
    void* fused_scratch_bf16;
    size_t fused_scratch_bytes;
    void const* transposed_candidates; // [hidden, rows_c]
    float* query_gradient;             // [rows_q, hidden], accumulated
    float gradient_scale;              // the loss passes 2 / live
};
// Returns the number of partial slots the launch fills: (column groups per tile) * rows_c / 64 / tiles_per_run.
uint32_t forward_partial_slots(uint32_t rows_c, uint32_t tiles_per_run);
uint32_t forward_quantities(uint32_t prefixes);
uint32_t forward_choose_tiles_per_run(uint32_t rows_q, uint32_t rows_c, int multiprocessors);
bool forward_fused_supported(uint32_t hidden, uint32_t prefixes);
uint32_t forward_choose_tiles_per_run_fused(uint32_t rows_q, uint32_t rows_c, int multiprocessors);
size_t forward_fused_scratch_bytes(uint32_t prefixes, uint32_t tiles_per_run, int multiprocessors);
constexpr int forward_trace_slots = 16;
void launch_forward(forward_arguments const& arguments, cudaStream_t stream);

struct backward_arguments {
    void const* gradient_cube_bf16;     // [K, rows_q, rows_c]
    void const* transposed_candidates;  // [hidden, rows_c]; may be null when the row-major block is given
    void const* candidates_row_major;   // [rows_c, hidden] as the block lies in memory; preferred when set (hidden >= 64)
    float* query_gradient;              // [rows_q, hidden], accumulated
    uint32_t* status;
    uint32_t rows_q, rows_c, hidden;
    ladder_host ladder;
    uint32_t split;                     // candidate-range splits (1: deterministic read-modify-write)
    float scale;                        // multiplies every product before accumulation (the loss passes 2 / live)
    uint64_t budget_ns;
};
void launch_backward(backward_arguments const& arguments, cudaStream_t stream);
// The backward launch's tile table for a shape, without launching: one {band, first channel, width, row blocks per CTA,
// first CTA of the tile's group, tiles in the group} per tile in grid order, and the grid's CTA count. A group's CTAs
// walk its tiles fastest, then the row blocks.
std::vector<std::array<uint32_t, 6>> backward_plan(uint32_t rows_q, ladder_host const& ladder, uint32_t split,
                                                    int multiprocessors, uint32_t* ctas);

void preload_loss_kernels();

// -------- projector tower (tower.cu) -----------------------------------------------------------------------------
// Elementwise passes between the tower's library GEMMs. bfloat16 matrices are row-major with a multiple of 8 columns.
// `partials` is scratch of tower_partial_blocks(rows) * columns floats; bias gradients leave as bfloat16 (the
// parameters' dtype), summed in float32 in a fixed order.
uint32_t tower_partial_blocks(uint32_t rows);
void launch_gelu_forward(void const* z_bf16, void* h_bf16, size_t scalars, int multiprocessors, cudaStream_t stream);
void launch_gelu_backward_bias(void const* upstream_bf16, void const* z_bf16, void* dz_bf16, float* partials, void* bias_grad_bf16,
                               uint32_t rows, uint32_t columns, cudaStream_t stream);
void launch_column_sums(void const* matrix_bf16, float* partials, void* sums_bf16, uint32_t rows, uint32_t columns,
                        cudaStream_t stream);

// -------- optimizer (optim.cu) -----------------------------------------------------------------------------------
// AdamW with decoupled weight decay over a list of tensors, eight per launch. Parameters and gradients bfloat16 or
// float32 (the same type for a tensor's pair), both moments float32. `step` counts from 1.
constexpr uint32_t adamw_max_tensors = 8;
struct adamw_tensor {
    void* param;
    void const* grad;
    float* exp_avg;
    float* exp_avg_sq;
    size_t count;
    uint32_t is_bf16;
    uint32_t vectorised; // set by the launcher: 16-byte loads apply
};
void launch_adamw(adamw_tensor const* tensors, uint32_t count, float lr, float beta1, float beta2, float eps, float decay,
                  uint64_t step, cudaStream_t stream);

// -------- bounds-checked debug build ----------------------------------------------------------------------------
// True in the build with -DSC_BOUNDS=1, in which kernels compare every computed global index with its limit. The
// readers copy out the first recorded miss of each translation unit (eight words, all zero when there was none; always
// zero in the ordinary build).
bool bounds_build();
void bounds_record_small(uint32_t* out);
void bounds_record_forward(uint32_t* out);
void bounds_record_backward(uint32_t* out);
void bounds_record_collectives(uint32_t* out);
void bounds_record_tower(uint32_t* out);
void bounds_record_optim(uint32_t* out);

// -------- oracle twin (oracle_cpu.cpp) ---------------------------------------------------------------------------
// Plain triple loop in float64; gradient [n, hidden]; out[0]=loss, out[1]=bias grad, out[2]=log-beta grad,
// out[4+k]=loss of prefix k.
void oracle_loops_f64(double const* world, size_t n, size_t hidden, ladder_host const& ladder, double beta, double bias,
                      uint32_t spec_code, double* gradient, double* out);

} // namespace sc
