// Forward tile kernel of the streamed Matryoshka sigmoid loss: scores a block of candidates against this rank's rows at
// every prefix, applies the sigmoid loss cell by cell, and leaves per band the suffix-summed gradient with respect to
// the raw dot product (bfloat16) plus per-row partial sums. Optionally the same launch pulls the NEXT peer's block
// from that peer's memory into local staging, so the NVLink transfer hides under this block's tensor-core work.
//
// Shape of the work. A tile is 128 query rows x 64 candidates. The hidden axis streams through shared memory in
// stages of 64 channels (TMA, 128-byte swizzle), widest channels first. Every band of the ladder owns one 64-column
// slot of tensor memory and the UMMAs of a 16-channel step accumulate into the slot of the band that contains the
// step, so each channel is multiplied exactly once (depth H per cell, where a sweep-and-subtract scheme spends up to
// 2H). The eight slots form a ring: while the epilogue warps drain the K slots of tile t, the issuing thread already
// fills the widest bands of tile t+1. The epilogue walks the bands narrowest first, adding each band's segment dots to
// a running prefix dot in registers, runs the cell math, parks the band's raw-dot gradients (without the factor
// beta / |q_k| that the row and band share) in the tensor-memory slot the dots came from, and then walks the bands
// widest first, two at a time, to form the suffix sums that go to the gradient cube. A tile's slots go back to the
// issuer in two steps: the two widest bands' as soon as the suffix pass has read them (the next tile's narrow bands
// wait for exactly those slots), the rest when the pass is done.
//
// Warp roles (608 threads): warps 0-15 epilogue (warp w owns tensor-memory lanes 32*(w%4).. and the 16 columns w/4 of
// the tile; four warps per scheduler keep the issue slots busy), warp 16 TMA producer, warp 17 UMMA issuer and
// tensor-memory owner (both run warp-wide, with the TMA / UMMA / commit instructions under one elected lane), warp 18
// peer pull (plain 16-byte loads from the peer's replica, plain stores to local staging; never a TMA load from another
// GPU's memory).
//
// A CTA walks work items (row strip, run of consecutive candidate tiles) in a fixed round-robin order and writes one
// partial record per (run, column quarter, row): the fold over runs happens later in run order, so the loss summands do
// not depend on scheduling.
//
// Parity: forward_tile_cuda_ and score_forward_row_ (scalingcontrasts.cuh:688-1040) and fold of its row partials;
// the staging copy of streamed_loss_t::score (scalingcontrasts.cuh:1262-1265) is what the pull warps replace.
#include <stdexcept>
#include <string>

#include "api.h"
#include "common.cuh"
#include "driver.h"

namespace sc {

namespace {

constexpr uint32_t fwd_rows = 128;
constexpr uint32_t fwd_cols = 64;
constexpr uint32_t fwd_depth = 64;
constexpr uint32_t fwd_max_stages = 6;
// Ladders of up to five prefixes leave room for six stages; longer ones keep more per-thread state and get five. The
// fused kernel shares the shared memory with the gradient GEMM's stages and keeps three.
__host__ __device__ constexpr uint32_t fwd_stages_for(uint32_t prefixes, bool fused) {
    return fused ? 3u : (prefixes <= 5 ? 6u : 5u);
}
constexpr uint32_t fwd_max_slots = 8;
// Tensor-memory slots of the score accumulators: all eight 64-column slots, or six when the last 128 columns hold the
// gradient GEMM's accumulator.
__host__ __device__ constexpr uint32_t fwd_slots_for(bool fused) { return fused ? 6u : 8u; }
constexpr uint32_t fwd_slot_columns = 64;
constexpr uint32_t fwd_tmem_columns = 512;
// The gradient GEMM that the fused kernel runs beside the scoring: 128 rows x up to 128 channels per accumulator, the
// candidate index as the K dimension in stages of 64, two stages of [128 rows of the gradient patch | 128 channels of
// the transposed candidates].
constexpr uint32_t fz_max_prefixes = 6;
constexpr uint32_t fz_depth = 64;
constexpr uint32_t fz_max_width = 128;
constexpr uint32_t fz_a_bytes = 128 * fz_depth * 2;
constexpr uint32_t fz_b_bytes = fz_max_width * fz_depth * 2;
constexpr uint32_t fz_stage_bytes = fz_a_bytes + fz_b_bytes;
constexpr uint32_t fz_stages = 2;
constexpr uint32_t fz_accumulator_column = 6 * fwd_slot_columns;
constexpr uint32_t fz_max_tiles = 48;
constexpr uint32_t fz_candidate_maps = 4; // boxes of 16, 32, 64 and 128 channels
constexpr uint32_t fz_max_tiles_per_run = 16;
#ifndef SC_FWD_EPILOGUE_WARPS
#define SC_FWD_EPILOGUE_WARPS 16
#endif
constexpr uint32_t fwd_epilogue_warps = SC_FWD_EPILOGUE_WARPS; // 16: four per scheduler at 96 registers; 8: two at 168
constexpr uint32_t fwd_epilogue_threads = fwd_epilogue_warps * 32;
constexpr uint32_t fwd_chunk_columns = 16;                                  // columns handled per tensor-memory load
constexpr uint32_t fwd_column_groups = fwd_epilogue_warps / 4;             // warps that share a lane quadrant
constexpr uint32_t fwd_warp_columns = fwd_cols / fwd_column_groups;        // columns of a tile that one warp owns
constexpr uint32_t fwd_warp_chunks = fwd_warp_columns / fwd_chunk_columns;
constexpr uint32_t fwd_producer_warp = fwd_epilogue_warps;
constexpr uint32_t fwd_mma_warp = fwd_epilogue_warps + 1;
constexpr uint32_t fwd_first_pull_warp = fwd_epilogue_warps + 2;
constexpr uint32_t fwd_pull_warps = 1;
constexpr uint32_t fz_mma_warp = fwd_epilogue_warps + 3; // fused kernel only; the pull warp doubles as its producer
__host__ __device__ constexpr uint32_t fwd_threads_for(bool fused) {
    return 32 * (fwd_epilogue_warps + 2 + fwd_pull_warps + (fused ? 1u : 0u));
}
constexpr uint32_t fwd_q_bytes = fwd_rows * fwd_depth * 2;
constexpr uint32_t fwd_c_bytes = fwd_cols * fwd_depth * 2;
constexpr uint32_t fwd_stage_bytes = fwd_q_bytes + fwd_c_bytes;
constexpr uint32_t fwd_tile_barriers = 8;
constexpr float log2_e = 1.4426950408889634f;
constexpr float easy_negative_limit = -8.0f; // (logit + bias) * log2(e) below this: e < 2^-8, the cubic series of log1p(e)
                                             // and e / (1 + e) are then exact to 2e-8 relative

struct fwd_tail {
    uint64_t stage_full[fwd_max_stages];
    uint64_t stage_empty[fwd_max_stages];
    // Tile t's accumulators have been read by every epilogue warp (index t % fwd_slots): `early` covers the two widest
    // bands, which the suffix pass reads first and whose slots the next tile's UMMAs want first; `late` covers the rest.
    uint64_t tile_early[fwd_max_slots];
    uint64_t tile_late[fwd_max_slots];
    uint64_t tile_full[fwd_tile_barriers];
    // Fused kernel: the gradient GEMM's stage ring, "this item's gradient patches are in memory" (one per scratch
    // buffer, an arrival per epilogue warp), and the hand-over of its single accumulator.
    uint64_t fz_stage_full[fz_stages];
    uint64_t fz_stage_empty[fz_stages];
    uint64_t fz_item_stored[2];
    uint64_t fz_accumulator_full;
    uint64_t fz_accumulator_empty;
    uint32_t tmem_base;
    uint32_t abort_flag;
};
constexpr uint32_t fwd_tail_bytes = (sizeof(fwd_tail) + 127) / 128 * 128;
// Per epilogue warp: [2 buffers][prefixes][16 columns] candidate inverse norms, then [2][8] tile maxima.
constexpr uint32_t fwd_norm_floats_per_warp = 2 * (8 * fwd_warp_columns + 8);
constexpr uint32_t fwd_norm_bytes = fwd_epilogue_warps * fwd_norm_floats_per_warp * 4;
// Per epilogue thread: inverse norm, loss and coefficient of every prefix, laid out [3 * prefixes][thread].
__host__ __device__ constexpr uint32_t fwd_state_bytes(uint32_t prefixes) { return 3 * prefixes * fwd_epilogue_threads * 4; }
// Per epilogue warp two staging buffers (one per band of a pair) of [32 rows][16 columns] bfloat16 for each of the warp's
// column chunks, from which the warp's patches of the gradient cube leave through TMA stores.
constexpr uint32_t fwd_store_patch_bytes = 32 * fwd_chunk_columns * 2;
constexpr uint32_t fwd_store_bytes = fwd_epilogue_warps * 2 * fwd_warp_chunks * fwd_store_patch_bytes;
__host__ __device__ constexpr uint32_t fwd_stage_region_bytes(uint32_t prefixes, bool fused) {
    return fwd_stages_for(prefixes, fused) * fwd_stage_bytes + (fused ? fz_stages * fz_stage_bytes : 0u);
}
__host__ __device__ constexpr uint32_t fwd_shared_bytes(uint32_t prefixes, bool fused) {
    return 1024 + fwd_stage_region_bytes(prefixes, fused) + fwd_store_bytes + fwd_tail_bytes + fwd_norm_bytes +
           fwd_state_bytes(prefixes);
}

struct fwd_params {
    float const* q_inv;
    float const* c_inv;
    float const* c_tile_max;
    __nv_bfloat16* cube;
    float* partials;
    uint32_t* status;
    uint32_t rows_q, rows_c, hidden;
    ladder_t ladder;
    uint32_t tiles_per_run, runs_per_strip, items;
    float beta, bias, weight;
    float const* scalars; // optional device copy of {beta, bias}: learnable values never visit the host
    uint64_t query_base, candidate_base;
    uint32_t spec_code;
    uint64_t budget_ns;
    pull_request pull;
    unsigned long long* trace; // optional: phase cycle counters of CTA 0 (see forward_trace_slots in api.h)
    // One word per 64-channel chunk, one byte per 16-channel step of the chunk: non-zero when, walking the channels
    // downwards, the step is the first of a band (the topmost step, or the step just below a band's first channel).
    // Kept in the kernel's parameters so that the UMMA warp reads it through the uniform datapath. hidden <= 4096.
    uint32_t band_starts[64];
    // Fused kernel only. The gradient GEMM's channel tiles, one word each: band | first channel / 16 << 4 | width / 16
    // << 16; a tile never crosses a band edge, so its A operand is one band's patch.
    float* gradient;       // [rows_q, hidden] float32, accumulated with vector reductions
    float gradient_scale;  // the loss's 2 / live, applied as the accumulator leaves tensor memory
    uint32_t tile_count;
    uint32_t tiles[fz_max_tiles];
};

// The tensor maps only the fused kernel uses: one over the per-CTA scratch of gradient patches (box of 128 rows x 64
// candidates, 128-byte swizzle: the GEMM's A operand) and the transposed candidates under boxes of 16 << index channels.
struct fz_maps {
    CUtensorMap patches;
    CUtensorMap candidates[fz_candidate_maps];
};

// Phase timers, compiled in only with -DSC_FWD_TRACE=1 (a diagnostic build: the clock reads and their branches cost the
// epilogue a few percent of its issue slots). A role keeps its cycle counters in registers and adds them to the trace
// array once, when it is done, so that timing a phase costs a clock read and not a round trip to memory. Only CTA 0
// records. Without the flag the type is empty and the `trace` argument is ignored.
#ifndef SC_FWD_TRACE
#define SC_FWD_TRACE 0
#endif
#if SC_FWD_TRACE
struct phase_timer {
    long long since;
    unsigned long long cycles[4];
    bool on;
    __device__ __forceinline__ explicit phase_timer(fwd_params const& p) : since(0), cycles{0, 0, 0, 0}, on(false) {
#ifdef __CUDA_ARCH__
        on = p.trace != nullptr && blockIdx.x == 0;
        since = clock64();
#endif
    }
    __device__ __forceinline__ void only_if(bool keep) { on = on && keep; }
    // Adds the cycles since the last call to counter `which` (0..3 of this role) and restarts the clock.
    __device__ __forceinline__ void lap(int which) {
#ifdef __CUDA_ARCH__
        if (on) {
            long long const now = clock64();
            cycles[which] += static_cast<unsigned long long>(now - since);
            since = now;
        }
#endif
    }
    __device__ __forceinline__ void flush(fwd_params const& p, int first_slot, int count) {
        if (on)
            for (int i = 0; i < count; ++i) p.trace[first_slot + i] += cycles[i];
    }
};
#else
struct phase_timer {
    __device__ __forceinline__ explicit phase_timer(fwd_params const&) {}
    __device__ __forceinline__ void only_if(bool) {}
    __device__ __forceinline__ void lap(int) {}
    __device__ __forceinline__ void flush(fwd_params const&, int, int) {}
};
#endif

// ---- the cell math ----------------------------------------------------------------------------------------------
// Accumulators are kept without the 1/N weight: `g` sums -mask*z*(1-sigmoid(s)), `ga` sums that times (logit+bias),
// `loss` sums mask*softplus(-s); the weight is applied once when the partial record is written.
struct row_constants {
    float beta, bias, weight, raw_scale;
};

// The cell pass leaves each band's raw-dot gradients in tensor memory without the factor beta / |q_k| that is common to
// the row and the band; the suffix pass multiplies it in while it sums the bands. The norms kernel writes an inverse
// norm of 0 for a row of zero norm (factor 0, and its cosines are floored anyway); the cap only keeps a huge inverse
// norm of a tiny row from turning 0 * factor into a NaN.
__device__ __forceinline__ float row_factor(float beta, float inv_q) { return beta * fminf(inv_q, 1e30f); }

// Any cell: positives, the diagonal, floored cosines. Only tiles that touch the diagonal or hold a floored norm come here,
// so this is a real call (one copy of the code) rather than sixteen inlined ones: the kernel's hot loops stay small and
// contiguous in the instruction cache. Returns what the cell adds to each of the row's sums.
struct cell_outcome {
    float raw, loss, cell, cell_logit, coefficient;
};
__device__ __noinline__ cell_outcome cell_general(float prefix_dot, float inv_q, float inv_c, float beta, float bias,
                                                  float raw_scale, bool own, bool partner, uint32_t spec_code) {
    uint32_t const diagonal = (spec_code >> 1) & 3u; // 0 own, 1 negative, 2 skip
    float z = partner ? 1.0f : -1.0f;
    float mask = 1.0f;
    if (own) {
        if (diagonal == 0u) z = 1.0f;
        if (diagonal == 2u) mask = 0.0f;
    }
    float const inverse_denominator = fminf(inv_q * inv_c, 100.0f);
    bool const floored = inverse_denominator >= 100.0f;
    float const cosine = floored ? 0.0f : prefix_dot * inverse_denominator;
    float const logit = beta * (own ? 1.0f : cosine);
    float const a = logit + bias;
    float const s = z * a;
    float const d = fast_ex2(-fabsf(s) * log2_e);
    float const complement = (s >= 0.0f ? d : 1.0f) * fast_rcp(1.0f + d);
    float const cell = -mask * z * complement;
    float const raw = (own || floored) ? 0.0f : cell * inverse_denominator * raw_scale;
    return cell_outcome{raw, mask * (fmaxf(-s, 0.0f) + log1p_unit(d)), cell, cell * a, raw * prefix_dot};
}

__device__ __forceinline__ void tmem_store_16(uint32_t taddr, uint32_t const (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- roles ------------------------------------------------------------------------------------------------------
// The producer and UMMA roles are run by all 32 lanes of their warp, with only the TMA / UMMA / commit instructions
// themselves under the elected lane's predicate: loop counters, stage addresses and descriptors are then warp-uniform
// values the compiler can keep in uniform registers, which is where those instructions take their operands from. (Run
// by a single lane inside a divergent branch, every operand would cross from a vector to a uniform register first.)
// Every lane waits; the answer is the same in every lane.
// Their waits sleep between attempts (`sleep_ns`; 0 polls back to back): a helper warp shares its scheduler with four
// epilogue warps, and a warp that polls an mbarrier without pause issues about as many instructions as one of them.
#ifndef SC_FWD_HELPER_SLEEP
#define SC_FWD_HELPER_SLEEP 1
#endif
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, wait_context const& ctx, uint32_t site,
                                               uint32_t detail, uint32_t sleep_ns = 0) {
    if (SC_FWD_HELPER_SLEEP && sleep_ns != 0u)
        return __all_sync(0xFFFFFFFFu, mbar_wait_relaxed(bar, parity, ctx, site, detail, sleep_ns));
    return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, ctx, site, detail));
}
constexpr uint32_t sleep_producer_ns = 1000; // stages ahead of the issuer: nothing waits for this warp's wake-up
constexpr uint32_t sleep_issuer_ns = 100;    // the epilogue may be waiting for the tile these UMMAs finish
constexpr uint32_t sleep_gemm_ns = 500;      // the fused kernel's gradient GEMM runs a whole item behind

__device__ __forceinline__ void producer_role(CUtensorMap const* q_map, CUtensorMap const* c_map, fwd_params const& p,
                                              uint32_t stages_base, fwd_tail* tail, wait_context const& ctx,
                                              uint32_t const stages) {
    bool const elected = elect_one();
    uint32_t stage = 0, phase = 0;
    uint32_t const chunks = p.hidden / fwd_depth;
    phase_timer timer(p);
    timer.only_if(elected);
    for (uint32_t item = blockIdx.x; item < p.items; item += gridDim.x) {
        uint32_t const strip = item / p.runs_per_strip, run = item % p.runs_per_strip;
        for (uint32_t t = 0; t < p.tiles_per_run; ++t) {
            uint32_t const column_tile = run * p.tiles_per_run + t;
            for (int chunk = static_cast<int>(chunks) - 1; chunk >= 0; --chunk) {
                timer.lap(0);
                if (!mbar_wait_warp(smem_u32(&tail->stage_empty[stage]), phase ^ 1u, ctx, site_fwd_stage_empty, item, sleep_producer_ns))
                    return;
                timer.lap(1);
                uint32_t const full = smem_u32(&tail->stage_full[stage]);
                uint32_t const destination = stages_base + stage * fwd_stage_bytes;
                if (elected) {
                    mbar_arrive_expect_tx(full, fwd_stage_bytes);
                    tma_load_2d(destination, q_map, full, chunk * static_cast<int>(fwd_depth), static_cast<int>(strip * fwd_rows));
                    tma_load_2d(destination + fwd_q_bytes, c_map, full, chunk * static_cast<int>(fwd_depth),
                                static_cast<int>(column_tile * fwd_cols));
                }
                __syncwarp();
                if (++stage == stages) stage = 0, phase ^= 1u;
            }
        }
    }
    timer.flush(p, 0, 2);
}

template <int prefixes_, bool fused_>
__device__ __forceinline__ void mma_role(fwd_params const& p, uint32_t stages_base, fwd_tail* tail, uint32_t tmem_base,
                                         wait_context const& ctx) {
    constexpr uint32_t fwd_slots = fwd_slots_for(fused_);
    constexpr uint32_t idesc = umma_idesc_bf16(fwd_rows, fwd_cols);
    constexpr uint32_t descriptor_high = (1024u >> 4) | (1u << 14) | (2u << 29); // stride 1024 B, version 1, 128-byte swizzle
    bool const elected = elect_one();
    uint32_t const chunks = p.hidden / fwd_depth;
    uint32_t const low_base = ((stages_base & 0x3FFFFu) >> 4) | (1u << 16);
    uint32_t stage = 0, phase = 0, unit = 0, tile_local = 0, seen_early = 0, seen_late = 0;
    phase_timer timer(p);
    timer.only_if(elected);
    for (uint32_t item = blockIdx.x; item < p.items; item += gridDim.x) {
        for (uint32_t t = 0; t < p.tiles_per_run; ++t) {
            uint32_t slot_address = 0, accumulate = 0;
            for (int chunk = static_cast<int>(chunks) - 1; chunk >= 0; --chunk) {
                uint32_t const starts = p.band_starts[chunk];
                timer.lap(0);
                if (!mbar_wait_warp(smem_u32(&tail->stage_full[stage]), phase, ctx, site_fwd_stage_full, tile_local, sleep_issuer_ns))
                    return;
                timer.lap(1);
                tcgen05_fence_after();
                uint32_t const low = low_base + stage * (fwd_stage_bytes >> 4);
#pragma unroll
                for (int sub = 3; sub >= 0; --sub) {
                    if ((starts >> (8 * sub)) & 0xFFu) {
                        // The slot's last user was unit - fwd_slots, band `rank` (counted from the widest) of tile `needed`;
                        // the epilogue must have read it out. Releases are observed here strictly in tile order, per
                        // barrier array, so a barrier's parity can never be a full turn ahead of the one waited for: tile
                        // X + fwd_slots cannot even be issued before tile X's release has been seen.
                        uint32_t const slot = unit % fwd_slots;
                        if (unit >= fwd_slots) {
                            uint32_t const needed = (unit - fwd_slots) / prefixes_, rank = (unit - fwd_slots) % prefixes_;
                            timer.lap(0);
                            if (rank < 2) {
                                while (seen_early <= needed) {
                                    if (!mbar_wait_warp(smem_u32(&tail->tile_early[seen_early % fwd_slots]),
                                                        (seen_early / fwd_slots) & 1u, ctx, site_fwd_slot_empty, unit, sleep_issuer_ns))
                                        return;
                                    ++seen_early;
                                }
                            } else {
                                while (seen_late <= needed) {
                                    if (!mbar_wait_warp(smem_u32(&tail->tile_late[seen_late % fwd_slots]),
                                                        (seen_late / fwd_slots) & 1u, ctx, site_fwd_slot_empty, unit, sleep_issuer_ns))
                                        return;
                                    ++seen_late;
                                }
                            }
                            timer.lap(2);
                        }
                        tcgen05_fence_after();
                        slot_address = tmem_base + slot * fwd_slot_columns;
                        accumulate = 0;
                        ++unit;
                    }
                    uint32_t const q_low = low + static_cast<uint32_t>(sub) * 2u; // 32 bytes per 16-channel step
                    uint64_t q_descriptor, c_descriptor;
                    asm("mov.b64 %0, {%1, %2};" : "=l"(q_descriptor) : "r"(q_low), "r"(descriptor_high));
                    asm("mov.b64 %0, {%1, %2};" : "=l"(c_descriptor) : "r"(q_low + (fwd_q_bytes >> 4)), "r"(descriptor_high));
                    if (elected) umma_bf16(slot_address, q_descriptor, c_descriptor, idesc, accumulate);
                    accumulate = 1;
                }
                if (elected) umma_commit(smem_u32(&tail->stage_empty[stage]));
                __syncwarp();
                if (++stage == fwd_stages_for(prefixes_, fused_)) stage = 0, phase ^= 1u;
            }
            if (elected) umma_commit(smem_u32(&tail->tile_full[tile_local % fwd_tile_barriers]));
            __syncwarp();
            ++tile_local;
        }
    }
    timer.flush(p, 2, 3);
}

// Position of a CTA in its fixed walk over (work item, tile of the run). The item's strip and run are carried along, so
// the division by the runtime run count happens once per item and not once per tile.
struct tile_cursor {
    uint32_t item, t, strip, run;
    __device__ __forceinline__ static tile_cursor at(fwd_params const& p, uint32_t item) {
        return tile_cursor{item, 0, item / p.runs_per_strip, item % p.runs_per_strip};
    }
    __device__ __forceinline__ bool valid(fwd_params const& p) const { return item < p.items; }
    __device__ __forceinline__ tile_cursor next(fwd_params const& p) const {
        return t + 1 < p.tiles_per_run ? tile_cursor{item, t + 1, strip, run} : at(p, item + gridDim.x);
    }
    __device__ __forceinline__ uint32_t column_tile(fwd_params const& p) const { return run * p.tiles_per_run + t; }
};

// Epilogue warps: warp w owns tensor-memory lanes 32*(w%4).. (a quarter of the tile's rows) and the column group w/4 of
// the tile (16 columns each with sixteen warps). The loop over prefixes is rolled (small code, few registers, four
// warps per scheduler): a prefix's segment dots come out of tensor memory, its raw-dot gradients go back into the same
// slot, and a second rolled pass reads them widest first, in pairs, to form the suffix sums. Per-thread sums that are
// indexed by prefix live in shared memory.
// Fused kernel: one warp's share of a finished accumulator of the gradient GEMM, added to the owner's rows. The
// accumulator is [128 rows x width channels]; the warp owns the 32 rows of its lane quadrant and every fourth 16-column
// chunk, starting at its column group. A real call: the code exists once and the hot loops keep their registers.
__device__ __noinline__ void fz_drain_chunks(float* destination, uint32_t chunks, uint32_t accumulator, uint32_t group,
                                             float scale) {
    for (uint32_t chunk = group; chunk < chunks; chunk += fwd_column_groups) {
        uint32_t values[16];
        tmem_load_16(accumulator + chunk * 16u, values);
        tmem_load_wait();
#pragma unroll
        for (int v = 0; v < 4; ++v)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(destination + chunk * 16u + 4 * v),
                         "f"(scale * __uint_as_float(values[4 * v])), "f"(scale * __uint_as_float(values[4 * v + 1])),
                         "f"(scale * __uint_as_float(values[4 * v + 2])), "f"(scale * __uint_as_float(values[4 * v + 3]))
                         : "memory");
    }
}

template <int prefixes_, bool fused_>
__device__ __forceinline__ void epilogue_role(CUtensorMap const* cube_map, fwd_params const& p, fwd_tail* tail,
                                              uint32_t store_base, float* norm_staging, float* thread_state,
                                              uint32_t tmem_base, wait_context const& ctx, uint32_t warp, uint32_t lane) {
    constexpr uint32_t fwd_slots = fwd_slots_for(fused_);
    constexpr int columns = fwd_chunk_columns;
    constexpr int chunks = fwd_warp_chunks;
    constexpr int warp_columns = fwd_warp_columns;
    constexpr int norm_count = prefixes_ * warp_columns;
    constexpr int ahead_count = (norm_count + 31) / 32;
    uint32_t const quadrant = warp % 4, group = warp / 4;
    uint32_t const row_local = quadrant * 32 + lane;
    uint32_t const lane_base = tmem_base + ((quadrant * 32u) << 16) + group * warp_columns;
    uint32_t const column_tiles = p.rows_c / fwd_cols;
    uint32_t const quantities = 2 + 2 * prefixes_;
    float const beta = p.scalars != nullptr ? __ldg(p.scalars) : p.beta;
    float const bias = p.scalars != nullptr ? __ldg(p.scalars + 1) : p.bias;
    row_constants const constants{beta, bias, p.weight, beta};
    float* const staged_norms = norm_staging + warp * fwd_norm_floats_per_warp; // [2][8][warp_columns]
    float* const staged_max = staged_norms + 2 * 8 * warp_columns;              // [2][8]
    float* const mine = thread_state + threadIdx.x;                             // [3 * prefixes_] strided by the thread count
    uint32_t tile_local = 0, buffer = 0;
    uint32_t const warp_store_base = store_base + warp * (2u * chunks) * fwd_store_patch_bytes;

    tile_cursor cursor = tile_cursor::at(p, blockIdx.x);
    if (!cursor.valid(p)) return;
    // Norms of a tile's candidates are fetched one tile ahead into registers and parked in this warp's shared-memory
    // buffer, so the cell loop reads them with broadcast shared loads instead of waiting on global memory.
    float ahead[ahead_count], ahead_max = 0.0f;
    auto fetch = [&](tile_cursor const& where) {
        uint32_t const column_tile = where.column_tile(p);
#pragma unroll
        for (int j = 0; j < ahead_count; ++j) {
            uint32_t const index = lane + 32 * j; // (prefix, column) = (index / warp_columns, index % warp_columns)
            if (index < norm_count &&
                SC_IN_BOUNDS(static_cast<size_t>(index / warp_columns) * p.rows_c + column_tile * fwd_cols + group * warp_columns +
                                 index % warp_columns,
                             static_cast<size_t>(prefixes_) * p.rows_c))
                ahead[j] = __ldg(p.c_inv + static_cast<size_t>(index / warp_columns) * p.rows_c + column_tile * fwd_cols +
                                 group * warp_columns + index % warp_columns);
        }
        if (lane < prefixes_ &&
            SC_IN_BOUNDS(static_cast<size_t>(lane) * column_tiles + column_tile, static_cast<size_t>(prefixes_) * column_tiles))
            ahead_max = __ldg(p.c_tile_max + static_cast<size_t>(lane) * column_tiles + column_tile);
    };
    auto park = [&](uint32_t into) {
#pragma unroll
        for (int j = 0; j < ahead_count; ++j) {
            uint32_t const index = lane + 32 * j;
            if (index < norm_count) staged_norms[into * 8 * warp_columns + index] = ahead[j];
        }
        if (lane < prefixes_) staged_max[into * 8 + lane] = ahead_max;
        __syncwarp();
    };
    fetch(cursor);
    park(0);

    float g = 0.0f, ga = 0.0f;
    uint32_t row = 0;
    uint64_t global_row = 0;
    phase_timer timer(p);
    timer.only_if(threadIdx.x == 0);

    // Fused kernel: the gradient GEMM of a finished item runs on the tensor cores while these warps score the next
    // item. Its accumulators (one per channel tile, `tile_count` per item, in item order) are drained here: whichever
    // are ready at the top of a tile, and, before the scratch buffer of item n - 1 is written again by item n + 1,
    // everything up to item n - 1 (by then long done). `drained` counts the accumulators this warp has taken; the
    // GEMM does not start accumulator u + 1 before all sixteen warps have taken u, so the barrier's parity is exact.
    uint32_t items_done = 0, drained = 0;
    auto drain = [&](uint32_t limit, bool blocking) -> bool {
        while (drained < limit) {
            uint32_t const full = smem_u32(&tail->fz_accumulator_full);
            if (blocking) {
                if (!mbar_wait(full, drained & 1u, ctx, site_fz_accumulator_full, drained)) return false;
            } else if (__shfl_sync(0xFFFFFFFFu, mbar_test_wait(full, drained & 1u) ? 1 : 0, 0) == 0) {
                break;
            }
            tcgen05_fence_after();
            uint32_t const item = blockIdx.x + (drained / p.tile_count) * gridDim.x;
            uint32_t const word = p.tiles[drained % p.tile_count];
            float* const destination = p.gradient +
                                       (static_cast<size_t>(item / p.runs_per_strip) * fwd_rows + row_local) * p.hidden +
                                       ((word >> 4) & 0xFFFu) * 16u;
            if (SC_WARP_IN_BOUNDS((static_cast<size_t>(item / p.runs_per_strip) * fwd_rows + row_local) * p.hidden +
                                      ((word >> 4) & 0xFFFu) * 16u + (word >> 16) * 16u - 1,
                                  static_cast<size_t>(p.rows_q) * p.hidden))
                fz_drain_chunks(destination, word >> 16, tmem_base + ((quadrant * 32u) << 16) + fz_accumulator_column, group,
                            p.gradient_scale);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tail->fz_accumulator_empty));
            ++drained;
        }
        return true;
    };

    while (cursor.valid(p)) {
        tile_cursor const following = cursor.next(p);
        bool const more = following.valid(p);
        if (more) fetch(following);
        if constexpr (fused_) drain(items_done * p.tile_count, false);
        uint32_t const strip = cursor.strip, run = cursor.run;
        if (cursor.t == 0) {
            row = strip * fwd_rows + row_local;
            global_row = p.query_base + row;
#pragma unroll
            for (int k = 0; k < prefixes_; ++k) {
                mine[k * fwd_epilogue_threads] = __ldg(p.q_inv + static_cast<size_t>(k) * p.rows_q + row);
                mine[(prefixes_ + k) * fwd_epilogue_threads] = 0.0f;
                mine[(2 * prefixes_ + k) * fwd_epilogue_threads] = 0.0f;
            }
            g = 0.0f, ga = 0.0f;
        }
        uint32_t const column_tile = cursor.column_tile(p);
        uint32_t const column = column_tile * fwd_cols + group * warp_columns;
        float const* const norms_now = staged_norms + buffer * 8 * warp_columns;
        // Is every cell of this warp's patch a plain negative off the cosine floor? The patch is special when its columns
        // come within one of its rows (a row's own copy, or its pair partner next to it), decided per warp so that a
        // tile on the diagonal sends only the patches the diagonal crosses through the general cell.
        uint64_t const first_row = p.query_base + static_cast<uint64_t>(strip) * fwd_rows + quadrant * 32u;
        uint64_t const first_column = p.candidate_base + column;
        bool special = first_column < first_row + 32u + 1 && first_row < first_column + warp_columns + 1;
#pragma unroll
        for (int k = 0; k < prefixes_; ++k) special |= mine[k * fwd_epilogue_threads] * staged_max[buffer * 8 + k] >= 100.0f;
        special = __any_sync(0xFFFFFFFFu, special);

        timer.lap(0);
        if (!mbar_wait(smem_u32(&tail->tile_full[tile_local % fwd_tile_barriers]), (tile_local / fwd_tile_barriers) & 1u, ctx,
                       site_fwd_tile_full, tile_local))
            return;
        tcgen05_fence_after();
        timer.lap(1);

        uint32_t const first_unit = tile_local * prefixes_;
        pair_t prefix[chunks][columns / 2];
#pragma unroll
        for (int h = 0; h < chunks; ++h)
#pragma unroll
            for (int c = 0; c < columns / 2; ++c) prefix[h][c] = pack2(0.0f, 0.0f);
        pair_t const bias2 = pack2(bias, bias);
#pragma unroll 1
        for (int k = 0; k < prefixes_; ++k) {
            uint32_t const address = lane_base + ((first_unit + (prefixes_ - 1 - k)) % fwd_slots) * fwd_slot_columns;
            uint32_t d[chunks][columns];
#pragma unroll
            for (int h = 0; h < chunks; ++h) tmem_load_16(address + h * columns, d[h]);
            // Candidate norms are read from the warp's staging buffer pair by pair, right where they are used (broadcast
            // shared loads), which keeps registers free for interleaving the cells.
            pair_t const* const inv_c = reinterpret_cast<pair_t const*>(norms_now + k * warp_columns);
            float const inv_q = mine[k * fwd_epilogue_threads];
            float const row_beta = row_factor(beta, inv_q);
            float loss = 0.0f, coefficient = 0.0f;
            tmem_load_wait();
            if (!special) {
                pair_t const row_beta2 = pack2(row_beta, row_beta);
                // First every cell's e = exp(logit + bias), computed in base two (the scale and the bias carry log2(e), so
                // the exponential is a single MUFU), and the largest logit + bias of the thread's cells. Where the warp's
                // patch is all easy negatives (every logit + bias below the limit, which is all but the hardest cells) e
                // is the decay exp(-|logit + bias|) and the rest is a few packed multiply-adds: log1p(e) = e - e^2/2 +
                // e^3/3 and 1 - sigmoid = e / (1 + e) = e - e^2 + e^3, both exact to better than 2e-8 relative below the
                // limit. Otherwise the general form runs: the decay with the absolute value, reciprocal, select by sign,
                // the full log1p polynomial, the hinge.
                pair_t const row_beta2_binary = pack2(row_beta * log2_e, row_beta * log2_e);
                pair_t const bias2_binary = pack2(bias * log2_e, bias * log2_e);
                pair_t decay[chunks][columns / 2];
                float largest0 = -INFINITY, largest1 = -INFINITY;
#pragma unroll
                for (int h = 0; h < chunks; ++h) {
#pragma unroll
                    for (int c = 0; c < columns / 2; ++c) {
                        prefix[h][c] = add2(prefix[h][c], pack2(__uint_as_float(d[h][2 * c]), __uint_as_float(d[h][2 * c + 1])));
                        pair_t const a = fma2(prefix[h][c], mul2(inv_c[h * (columns / 2) + c], row_beta2_binary), bias2_binary);
                        float a0, a1;
                        unpack2(a, a0, a1);
                        decay[h][c] = pack2(fast_ex2(a0), fast_ex2(a1));
                        largest0 = fmaxf(largest0, a0), largest1 = fmaxf(largest1, a1);
                    }
                }
                float lo, hi, band_g;
                pair_t loss2 = pack2(0.0f, 0.0f), coefficient2 = pack2(0.0f, 0.0f), g2 = pack2(0.0f, 0.0f);
                if (__all_sync(0xFFFFFFFFu, fmaxf(largest0, largest1) < easy_negative_limit)) {
                    pair_t singles = pack2(0.0f, 0.0f), squares = pack2(0.0f, 0.0f), cubes = pack2(0.0f, 0.0f);
                    pair_t const minus_one = pack2(-1.0f, -1.0f);
#pragma unroll
                    for (int h = 0; h < chunks; ++h) {
#pragma unroll
                        for (int c = 0; c < columns / 2; ++c) {
                            pair_t const e = decay[h][c];
                            pair_t const square = mul2(e, e);
                            singles = add2(singles, e);
                            squares = add2(squares, square);
                            cubes = fma2(square, e, cubes);
                            pair_t const complement = fma2(square, add2(e, minus_one), e);
                            pair_t const raw = mul2(complement, inv_c[h * (columns / 2) + c]);
                            coefficient2 = fma2(raw, prefix[h][c], coefficient2);
                            float raw0, raw1;
                            unpack2(raw, raw0, raw1);
                            d[h][2 * c] = __float_as_uint(raw0), d[h][2 * c + 1] = __float_as_uint(raw1);
                        }
                    }
                    // Both sums are combinations of the power sums: loss e - e^2/2 + e^3/3, complement e - e^2 + e^3.
                    loss2 = fma2(squares, pack2(-0.5f, -0.5f), singles);
                    loss2 = fma2(cubes, pack2(1.0f / 3.0f, 1.0f / 3.0f), loss2);
                    g2 = add2(fma2(squares, minus_one, singles), cubes);
                } else {
#pragma unroll
                    for (int h = 0; h < chunks; ++h) {
#pragma unroll
                        for (int c = 0; c < columns / 2; ++c) {
                            pair_t const scale = mul2(inv_c[h * (columns / 2) + c], row_beta2);
                            float a0, a1, e0, e1, s0, s1;
                            unpack2(fma2(prefix[h][c], scale, bias2), a0, a1);
                            e0 = fast_ex2(-fabsf(a0) * log2_e), e1 = fast_ex2(-fabsf(a1) * log2_e);
                            pair_t const e = pack2(e0, e1);
                            unpack2(add2(e, pack2(1.0f, 1.0f)), s0, s1);
                            pair_t const complement =
                                mul2(pack2(a0 >= 0.0f ? 1.0f : e0, a1 >= 0.0f ? 1.0f : e1), pack2(fast_rcp(s0), fast_rcp(s1)));
                            loss2 = add2(fma2(log1p_ratio2(e), e, loss2), pack2(fmaxf(a0, 0.0f), fmaxf(a1, 0.0f)));
                            g2 = add2(g2, complement);
                            pair_t const raw = mul2(complement, inv_c[h * (columns / 2) + c]);
                            coefficient2 = fma2(raw, prefix[h][c], coefficient2);
                            float raw0, raw1;
                            unpack2(raw, raw0, raw1);
                            d[h][2 * c] = __float_as_uint(raw0), d[h][2 * c + 1] = __float_as_uint(raw1);
                        }
                    }
                }
                unpack2(loss2, lo, hi);
                loss = lo + hi;
                unpack2(coefficient2, lo, hi);
                coefficient = row_beta * (lo + hi);
                unpack2(g2, lo, hi);
                band_g = lo + hi;
                g += band_g;
                // sum of complement * (logit + bias) = sum of raw * dot + bias * sum of complement
                ga += fmaf(bias, band_g, coefficient);
            } else {
                // Which of this warp's columns, if any, is the row's own copy or its pair partner.
                int64_t const first = static_cast<int64_t>(p.candidate_base + column);
                int64_t const own_at = static_cast<int64_t>(global_row) - first;
                int64_t const partner_at = static_cast<int64_t>(global_row ^ 1ull) - first;
                int const own_column = own_at >= 0 && own_at < warp_columns ? static_cast<int>(own_at) : -1;
                int const partner_column =
                    (p.spec_code & 1u) != 0u && partner_at >= 0 && partner_at < warp_columns ? static_cast<int>(partner_at) : -1;
                float const without_row_factor = row_beta != 0.0f ? __fdividef(1.0f, row_beta) : 0.0f;
#pragma unroll
                for (int h = 0; h < chunks; ++h) {
#pragma unroll
                    for (int c = 0; c < columns / 2; ++c) {
                        prefix[h][c] = add2(prefix[h][c], pack2(__uint_as_float(d[h][2 * c]), __uint_as_float(d[h][2 * c + 1])));
                        float dot0, dot1, norm0, norm1;
                        unpack2(prefix[h][c], dot0, dot1);
                        unpack2(inv_c[h * (columns / 2) + c], norm0, norm1);
                        int const at = h * columns + 2 * c;
                        cell_outcome const first_cell = cell_general(dot0, inv_q, norm0, constants.beta, constants.bias,
                                                                     constants.raw_scale, at == own_column, at == partner_column,
                                                                     p.spec_code);
                        cell_outcome const second_cell =
                            cell_general(dot1, inv_q, norm1, constants.beta, constants.bias, constants.raw_scale,
                                         at + 1 == own_column, at + 1 == partner_column, p.spec_code);
                        d[h][2 * c] = __float_as_uint(first_cell.raw * without_row_factor);
                        d[h][2 * c + 1] = __float_as_uint(second_cell.raw * without_row_factor);
                        loss += first_cell.loss + second_cell.loss;
                        g += first_cell.cell + second_cell.cell;
                        ga += first_cell.cell_logit + second_cell.cell_logit;
                        coefficient += first_cell.coefficient + second_cell.coefficient;
                    }
                }
            }
#pragma unroll
            for (int h = 0; h < chunks; ++h) tmem_store_16(address + h * columns, d[h]);
            mine[(prefixes_ + k) * fwd_epilogue_threads] += loss;
            mine[(2 * prefixes_ + k) * fwd_epilogue_threads] += coefficient;
        }
        tmem_store_wait();
        timer.lap(2);
        // Suffix sums, widest band first: band k's gradient cube holds the sum over bands >= k.
        pair_t running[chunks][columns / 2];
#pragma unroll
        for (int h = 0; h < chunks; ++h)
#pragma unroll
            for (int c = 0; c < columns / 2; ++c) running[h][c] = pack2(0.0f, 0.0f);
        // Bands are taken two at a time: both loads are in flight together, both patches are staged behind one proxy
        // fence, and both leave in one bulk group, so a tile pays the load -> convert -> stage -> fence -> store latency
        // chain three times for five bands instead of five times. A [32 rows x 16 columns] patch of a band goes to one of
        // the warp's staging buffers (32 bytes per row) and leaves as a TMA store issued by lane 0, so no load/store-unit
        // instruction touches global memory and no other warp is waited for. Before the buffers are rewritten, the
        // stores that read them (the previous group) must have finished reading.
        auto band_address = [&](int band) {
            return lane_base + ((first_unit + (prefixes_ - 1 - band)) % fwd_slots) * fwd_slot_columns;
        };
        auto fold_and_pack = [&](uint32_t const (&d)[chunks][columns], int band, uint32_t (&packed)[chunks][columns / 2]) {
            float const factor = row_factor(beta, mine[band * fwd_epilogue_threads]);
            pair_t const factor2 = pack2(factor, factor);
#pragma unroll
            for (int h = 0; h < chunks; ++h)
#pragma unroll
                for (int c = 0; c < columns / 2; ++c) {
                    running[h][c] =
                        fma2(pack2(__uint_as_float(d[h][2 * c]), __uint_as_float(d[h][2 * c + 1])), factor2, running[h][c]);
                    float lo, hi;
                    unpack2(running[h][c], lo, hi);
                    packed[h][c] = pack_bf16x2(lo, hi);
                }
        };
        auto stage_patches = [&](uint32_t const (&packed)[chunks][columns / 2], uint32_t half) {
#pragma unroll
            for (int h = 0; h < chunks; ++h) {
                uint32_t const patch = warp_store_base + (half * chunks + h) * fwd_store_patch_bytes + lane * 32u;
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(patch), "r"(packed[h][0]), "r"(packed[h][1]),
                             "r"(packed[h][2]), "r"(packed[h][3]) : "memory");
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(patch + 16u), "r"(packed[h][4]), "r"(packed[h][5]),
                             "r"(packed[h][6]), "r"(packed[h][7]) : "memory");
            }
        };
        // Where the warp's patches go: into the block's gradient cube at the tile's place, or (fused kernel) into this
        // CTA's scratch buffer of the item, [band][128 rows][tiles_per_run * 64 candidates], at the tile's place in the run.
        uint32_t const store_x = fused_ ? cursor.t * fwd_cols + group * warp_columns : column;
        uint32_t const store_y = fused_ ? quadrant * 32u : strip * fwd_rows + quadrant * 32u;
        uint32_t const store_z = fused_ ? (blockIdx.x * 2u + (items_done & 1u)) * prefixes_ : 0u;
        auto send_patches = [&](uint32_t half, int band) {
#pragma unroll
            for (int h = 0; h < chunks; ++h)
                asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                                 reinterpret_cast<uint64_t>(cube_map)),
                             "r"(warp_store_base + (half * chunks + h) * fwd_store_patch_bytes), "r"(store_x + h * columns),
                             "r"(store_y), "r"(store_z + band)
                             : "memory");
        };
        auto release = [&](uint64_t* barriers) {
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&barriers[tile_local % fwd_slots]));
        };
        int k = prefixes_ - 1;
#pragma unroll 1
        for (; k >= 1; k -= 2) {
            uint32_t upper[chunks][columns], lower[chunks][columns];
#pragma unroll
            for (int h = 0; h < chunks; ++h) tmem_load_16(band_address(k) + h * columns, upper[h]);
#pragma unroll
            for (int h = 0; h < chunks; ++h) tmem_load_16(band_address(k - 1) + h * columns, lower[h]);
            tmem_load_wait();
            if (k == prefixes_ - 1) release(tail->tile_early);
            uint32_t packed_upper[chunks][columns / 2], packed_lower[chunks][columns / 2];
            fold_and_pack(upper, k, packed_upper);
            fold_and_pack(lower, k - 1, packed_lower);
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            __syncwarp();
            stage_patches(packed_upper, 0);
            stage_patches(packed_lower, 1);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                send_patches(0, k);
                send_patches(1, k - 1);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        }
        if (k == 0) {
            uint32_t last[chunks][columns];
#pragma unroll
            for (int h = 0; h < chunks; ++h) tmem_load_16(band_address(0) + h * columns, last[h]);
            tmem_load_wait();
            if (prefixes_ == 1) release(tail->tile_early);
            uint32_t packed_last[chunks][columns / 2];
            fold_and_pack(last, 0, packed_last);
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            __syncwarp();
            stage_patches(packed_last, 0);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                send_patches(0, 0);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        }
        timer.lap(3);
        // This warp is done with the tile's slots.
        release(tail->tile_late);
        if (more) park(buffer ^ 1u);
        if (cursor.t + 1 == p.tiles_per_run) {
            // One partial record per (run, column group, row); the 1/N weight and the mirror cell's factor two go in here.
            uint32_t const slot = run * fwd_column_groups + group;
            float* record = p.partials + static_cast<size_t>(slot) * quantities * p.rows_q + row;
            if (SC_IN_BOUNDS((static_cast<size_t>(slot) * quantities + quantities - 1) * p.rows_q + row,
                             static_cast<size_t>(p.runs_per_strip) * fwd_column_groups * quantities * p.rows_q)) {
            record[0] = p.weight * g;
            record[static_cast<size_t>(1) * p.rows_q] = p.weight * (ga - bias * g);
#pragma unroll
            for (int k = 0; k < prefixes_; ++k) {
                record[static_cast<size_t>(2 + k) * p.rows_q] = p.weight * mine[(prefixes_ + k) * fwd_epilogue_threads];
                record[static_cast<size_t>(2 + prefixes_ + k) * p.rows_q] =
                    2.0f * p.weight * mine[(2 * prefixes_ + k) * fwd_epilogue_threads];
            }
            }
            if constexpr (fused_) {
                // The item's patches of this warp are in memory once its bulk stores have completed (not merely been
                // read out of the staging buffers); then the gradient GEMM's producer may load them.
                if (lane == 0) {
                    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                    fence_proxy_async_all();
                    mbar_arrive(smem_u32(&tail->fz_item_stored[items_done & 1u]));
                }
                __syncwarp();
                ++items_done;
                // The next item writes the other scratch buffer, whose last reader was the GEMM of item items_done - 2.
                if (!drain((items_done - 1) * p.tile_count, true)) return;
            }
        }
        cursor = following;
        buffer ^= 1u;
        ++tile_local;
    }
    timer.flush(p, 5, 4);
    // The staging buffers must outlive the stores that read them.
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    if constexpr (fused_) drain(items_done * p.tile_count, true);
}

// ---- fused kernel: the gradient GEMM's two roles ------------------------------------------------------------------
// For every item this CTA has scored (in the same order), for every channel tile, the K loop over the item's candidates:
// A = the band's gradient patch [128 rows x 64 candidates] from this CTA's scratch buffer, B = the transposed candidates
// [width channels x 64 candidates]. Both K-major under the 128-byte swizzle.
__device__ __forceinline__ void fz_producer_role(fz_maps const* maps, fwd_params const& p, uint32_t stages_base,
                                                 fwd_tail* tail, wait_context const& ctx, uint32_t const prefixes) {
    bool const elected = elect_one();
    uint32_t stage = 0, phase = 0, local = 0;
    phase_timer timer(p);
    timer.only_if(elected);
    for (uint32_t item = blockIdx.x; item < p.items; item += gridDim.x, ++local) {
        uint32_t const buffer = local & 1u;
        timer.lap(0);
        if (!mbar_wait_warp(smem_u32(&tail->fz_item_stored[buffer]), (local >> 1) & 1u, ctx, site_fz_item_stored, item, sleep_producer_ns))
            return;
        timer.lap(1);
        fence_proxy_async_all();
        uint32_t const first_candidate = (item % p.runs_per_strip) * p.tiles_per_run * fwd_cols;
        for (uint32_t which = 0; which < p.tile_count; ++which) {
            uint32_t const word = p.tiles[which];
            uint32_t const band = word & 0xFu, channel0 = ((word >> 4) & 0xFFFu) * 16u, width = (word >> 16) * 16u;
            for (uint32_t block = 0; block < p.tiles_per_run; ++block) {
                timer.lap(0);
                if (!mbar_wait_warp(smem_u32(&tail->fz_stage_empty[stage]), phase ^ 1u, ctx, site_fz_stage_empty, which, sleep_gemm_ns))
                    return;
                timer.lap(2);
                uint32_t const full = smem_u32(&tail->fz_stage_full[stage]);
                uint32_t const destination = stages_base + stage * fz_stage_bytes;
                if (elected) {
                    mbar_arrive_expect_tx(full, fz_a_bytes + width * fz_depth * 2u);
                    tma_load_3d(destination, &maps->patches, full, static_cast<int>(block * fz_depth), 0,
                                static_cast<int>((blockIdx.x * 2u + buffer) * prefixes + band));
                    // Largest boxes first; 16 channels are 2048 bytes of the stage (rows of 128 bytes under the swizzle).
                    uint32_t done = 0;
#pragma unroll
                    for (int index = static_cast<int>(fz_candidate_maps) - 1; index >= 0; --index) {
                        uint32_t const box = 16u << index;
                        if (width - done >= box) {
                            tma_load_2d(destination + fz_a_bytes + done * 128u, &maps->candidates[index], full,
                                        static_cast<int>(first_candidate + block * fz_depth), static_cast<int>(channel0 + done));
                            done += box;
                        }
                    }
                }
                __syncwarp();
                if (++stage == fz_stages) stage = 0, phase ^= 1u;
            }
        }
    }
    timer.flush(p, 9, 3);
}

__device__ __forceinline__ void fz_mma_role(fwd_params const& p, uint32_t stages_base, fwd_tail* tail, uint32_t tmem_base,
                                            wait_context const& ctx) {
    constexpr uint32_t descriptor_high = (1024u >> 4) | (1u << 14) | (2u << 29); // stride 1024 B, version 1, 128-byte swizzle
    bool const elected = elect_one();
    uint32_t const low_base = ((stages_base & 0x3FFFFu) >> 4) | (1u << 16);
    uint32_t const accumulator = tmem_base + fz_accumulator_column;
    uint32_t stage = 0, phase = 0, unit = 0;
    phase_timer timer(p);
    timer.only_if(elected);
    for (uint32_t item = blockIdx.x; item < p.items; item += gridDim.x) {
        for (uint32_t which = 0; which < p.tile_count; ++which, ++unit) {
            uint32_t const idesc = umma_idesc_bf16(128, (p.tiles[which] >> 16) * 16u);
            // The accumulator's previous contents must have left tensor memory (an arrival per epilogue warp).
            timer.lap(0);
            if (unit != 0 &&
                !mbar_wait_warp(smem_u32(&tail->fz_accumulator_empty), (unit - 1) & 1u, ctx, site_fz_accumulator_empty, unit, sleep_gemm_ns))
                return;
            timer.lap(1);
            tcgen05_fence_after();
            for (uint32_t block = 0; block < p.tiles_per_run; ++block) {
                if (!mbar_wait_warp(smem_u32(&tail->fz_stage_full[stage]), phase, ctx, site_fz_stage_full, unit, sleep_gemm_ns)) return;
                timer.lap(2);
                tcgen05_fence_after();
                uint32_t const a_low = low_base + stage * (fz_stage_bytes >> 4);
                uint32_t const b_low = a_low + (fz_a_bytes >> 4);
#pragma unroll
                for (uint32_t step = 0; step < fz_depth / 16; ++step) {
                    uint64_t a_descriptor, b_descriptor;
                    asm("mov.b64 %0, {%1, %2};" : "=l"(a_descriptor) : "r"(a_low + step * 2u), "r"(descriptor_high));
                    asm("mov.b64 %0, {%1, %2};" : "=l"(b_descriptor) : "r"(b_low + step * 2u), "r"(descriptor_high));
                    if (elected) umma_bf16(accumulator, a_descriptor, b_descriptor, idesc, (block | step) != 0u ? 1u : 0u);
                }
                if (elected) umma_commit(smem_u32(&tail->fz_stage_empty[stage]));
                __syncwarp();
                if (++stage == fz_stages) stage = 0, phase ^= 1u;
            }
            if (elected) umma_commit(smem_u32(&tail->fz_accumulator_full));
            __syncwarp();
        }
    }
    timer.flush(p, 12, 3);
}

__device__ __forceinline__ void pull_role(pull_request const& request, uint32_t thread_in_role) {
    size_t const thread = static_cast<size_t>(blockIdx.x) * (fwd_pull_warps * 32) + thread_in_role;
    size_t const threads = static_cast<size_t>(gridDim.x) * (fwd_pull_warps * 32);
    for (int part = 0; part < 2; ++part) {
        size_t const vectors = request.bytes[part] / 16;
        if (vectors == 0) continue;
        uint4 const* src = static_cast<uint4 const*>(request.src[part]);
        uint4* dst = static_cast<uint4*>(request.dst[part]);
        size_t index = thread;
        for (; index + 7 * threads < vectors; index += 8 * threads) {
            uint4 held[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) held[u] = src[index + u * threads];
#pragma unroll
            for (int u = 0; u < 8; ++u) dst[index + u * threads] = held[u];
        }
        for (; index < vectors; index += threads) dst[index] = src[index];
    }
}

template <int prefixes_, bool fused_>
__global__ void __launch_bounds__(fwd_threads_for(fused_), 1)
    forward_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap c_map,
                   const __grid_constant__ CUtensorMap cube_map, const __grid_constant__ fz_maps gemm_maps,
                   const fwd_params p) {
    constexpr uint32_t fwd_slots = fwd_slots_for(fused_);
    constexpr uint32_t stages = fwd_stages_for(prefixes_, fused_);
    extern __shared__ uint8_t raw_shared[];
    uint32_t const raw_address = smem_u32(raw_shared);
    uint32_t const stages_base = (raw_address + 1023u) & ~1023u;
    uint32_t const gemm_stages_base = stages_base + stages * fwd_stage_bytes;
    uint32_t const store_base = stages_base + fwd_stage_region_bytes(prefixes_, fused_);
    fwd_tail* tail = reinterpret_cast<fwd_tail*>(raw_shared + (store_base - raw_address) + fwd_store_bytes);
    uint32_t const warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        tail->abort_flag = status_poisoned(p.status) ? 1u : 0u;
        for (uint32_t i = 0; i < fwd_max_stages; ++i) {
            mbar_init(smem_u32(&tail->stage_full[i]), 1);
            mbar_init(smem_u32(&tail->stage_empty[i]), 1);
        }
        for (uint32_t i = 0; i < fwd_slots; ++i) {
            mbar_init(smem_u32(&tail->tile_early[i]), fwd_epilogue_warps);
            mbar_init(smem_u32(&tail->tile_late[i]), fwd_epilogue_warps);
        }
        for (uint32_t i = 0; i < fwd_tile_barriers; ++i) mbar_init(smem_u32(&tail->tile_full[i]), 1);
        if constexpr (fused_) {
            for (uint32_t i = 0; i < fz_stages; ++i) {
                mbar_init(smem_u32(&tail->fz_stage_full[i]), 1);
                mbar_init(smem_u32(&tail->fz_stage_empty[i]), 1);
            }
            mbar_init(smem_u32(&tail->fz_item_stored[0]), fwd_epilogue_warps);
            mbar_init(smem_u32(&tail->fz_item_stored[1]), fwd_epilogue_warps);
            mbar_init(smem_u32(&tail->fz_accumulator_full), 1);
            mbar_init(smem_u32(&tail->fz_accumulator_empty), fwd_epilogue_warps);
        }
        fence_barrier_init();
    }
    __syncthreads();
    if (tail->abort_flag != 0u) return; // a poisoned status block: nothing was allocated, every thread leaves
    if (warp == fwd_mma_warp) {
        tmem_alloc(smem_u32(&tail->tmem_base), fwd_tmem_columns);
        tmem_relinquish();
    }
    if (warp == fwd_producer_warp && lane == 0) {
        tma_prefetch_descriptor(&q_map);
        tma_prefetch_descriptor(&c_map);
    }
    if constexpr (fused_) {
        if (warp == fwd_first_pull_warp && lane == 0) {
            tma_prefetch_descriptor(&gemm_maps.patches);
            for (uint32_t i = 0; i < fz_candidate_maps; ++i) tma_prefetch_descriptor(&gemm_maps.candidates[i]);
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    uint32_t const tmem_base = tail->tmem_base;
    wait_context const ctx{p.status, p.budget_ns, &tail->abort_flag};

    if (warp < fwd_epilogue_warps) {
        float* const norm_staging = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(tail) + fwd_tail_bytes);
        epilogue_role<prefixes_, fused_>(&cube_map, p, tail, store_base, norm_staging, norm_staging + fwd_norm_bytes / 4,
                                         tmem_base, ctx, warp, lane);
    } else if (warp == fwd_producer_warp) {
        producer_role(&q_map, &c_map, p, stages_base, tail, ctx, stages);
    } else if (warp == fwd_mma_warp) {
        mma_role<prefixes_, fused_>(p, stages_base, tail, tmem_base, ctx);
    } else if (warp == fwd_first_pull_warp) {
        // The pull is a short copy at the start of the launch; the gradient GEMM's first item is not ready before the
        // epilogue warps have scored a whole item, so the same warp serves both.
        pull_role(p.pull, threadIdx.x - fwd_first_pull_warp * 32);
        if constexpr (fused_) fz_producer_role(&gemm_maps, p, gemm_stages_base, tail, ctx, prefixes_);
    } else if (warp == fz_mma_warp) {
        if constexpr (fused_) fz_mma_role(p, gemm_stages_base, tail, tmem_base, ctx);
    }

    tcgen05_fence_before();
    __syncthreads();
    if (tail->abort_flag != 0u) {
        // Something gave up. Give copies and UMMAs that are still in flight a bounded time to land before the tensor
        // memory goes back.
        uint64_t const start = global_timer_ns();
        while (global_timer_ns() - start < 200000ull) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == fwd_mma_warp) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, fwd_tmem_columns);
    }
}

// ---- host side --------------------------------------------------------------------------------------------------
// Rows of `inner` bfloat16 values, `outer` of them, read in boxes under the 128-byte swizzle.
CUtensorMap const& operand_map(void const* base, uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer) {
    return cached_operand_map(base, inner, outer, box_inner, box_outer);
}

template <int prefixes_, bool fused_>
void launch_instance(CUtensorMap const& q_map, CUtensorMap const& c_map, CUtensorMap const& cube_map, fz_maps const& gemm_maps,
                     fwd_params const& p, int blocks, cudaStream_t stream) {
    // The attribute is per device; a process drives one GPU, but a second one costs only the repeat of a cheap call.
    static int prepared_device = -1;
    int device = 0;
    cudaGetDevice(&device);
    if (prepared_device != device) {
        require(cudaFuncSetAttribute(forward_kernel<prefixes_, fused_>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     fwd_shared_bytes(prefixes_, fused_)),
                "raising the forward kernel's shared memory");
        prepared_device = device;
    }
    forward_kernel<prefixes_, fused_><<<blocks, fwd_threads_for(fused_), fwd_shared_bytes(prefixes_, fused_), stream>>>(
        q_map, c_map, cube_map, gemm_maps, p);
}

template <bool fused_>
void launch_for_count(uint32_t count, CUtensorMap const& q_map, CUtensorMap const& c_map, CUtensorMap const& cube_map,
                      fz_maps const& gemm_maps, fwd_params const& p, int blocks, cudaStream_t stream) {
    switch (count) {
    case 1: launch_instance<1, fused_>(q_map, c_map, cube_map, gemm_maps, p, blocks, stream); break;
    case 2: launch_instance<2, fused_>(q_map, c_map, cube_map, gemm_maps, p, blocks, stream); break;
    case 3: launch_instance<3, fused_>(q_map, c_map, cube_map, gemm_maps, p, blocks, stream); break;
    case 4: launch_instance<4, fused_>(q_map, c_map, cube_map, gemm_maps, p, blocks, stream); break;
    case 5: launch_instance<5, fused_>(q_map, c_map, cube_map, gemm_maps, p, blocks, stream); break;
    case 6: launch_instance<6, fused_>(q_map, c_map, cube_map, gemm_maps, p, blocks, stream); break;
    default:
        if constexpr (!fused_) {
            if (count == 7) launch_instance<7, false>(q_map, c_map, cube_map, gemm_maps, p, blocks, stream);
            else launch_instance<8, false>(q_map, c_map, cube_map, gemm_maps, p, blocks, stream);
        }
        break;
    }
}

} // namespace

uint32_t forward_partial_slots(uint32_t rows_c, uint32_t tiles_per_run) {
    return fwd_column_groups * (rows_c / fwd_cols) / tiles_per_run;
}
uint32_t forward_quantities(uint32_t prefixes) { return 2 + 2 * prefixes; }

uint32_t forward_choose_tiles_per_run(uint32_t rows_q, uint32_t rows_c, int multiprocessors) {
    uint32_t const strips = rows_q / fwd_rows, column_tiles = rows_c / fwd_cols;
    uint32_t best = 1;
    for (uint32_t t = 1; t <= 32 && column_tiles % t == 0; t *= 2)
        if (static_cast<uint64_t>(strips) * (column_tiles / t) >= 6ull * static_cast<uint64_t>(multiprocessors)) best = t;
    return best;
}

bool forward_fused_supported(uint32_t hidden, uint32_t prefixes) { return prefixes <= fz_max_prefixes && hidden <= 4096; }

// A fused item is a run of tiles whose gradient patches one GEMM pass folds, adding a [128, hidden] float32 tile to the
// gradient once per item: runs of at least four tiles keep those additions rare, longer runs are taken while enough
// items remain to balance the GPU.
uint32_t forward_choose_tiles_per_run_fused(uint32_t rows_q, uint32_t rows_c, int multiprocessors) {
    uint32_t const strips = rows_q / fwd_rows, column_tiles = rows_c / fwd_cols;
    uint32_t best = 1;
    for (uint32_t t = 1; t <= fz_max_tiles_per_run && column_tiles % t == 0; t *= 2)
        if (t <= 4 || static_cast<uint64_t>(strips) * (column_tiles / t) >= 6ull * static_cast<uint64_t>(multiprocessors)) best = t;
    return best;
}

// Two buffers per CTA of [prefixes][128 rows][tiles_per_run * 64 candidates] bfloat16.
size_t forward_fused_scratch_bytes(uint32_t prefixes, uint32_t tiles_per_run, int multiprocessors) {
    return static_cast<size_t>(multiprocessors) * 2 * prefixes * fwd_rows * tiles_per_run * fwd_cols * 2;
}

void launch_forward(forward_arguments const& a, cudaStream_t stream) {
    if (a.rows_q % fwd_rows || a.rows_c % fwd_cols || a.hidden % fwd_depth || a.hidden > 4096)
        throw std::runtime_error("forward: rows must be multiples of 128 (queries) and 64 (candidates), hidden of 64 up to 4096");
    if (a.ladder.count < 1 || a.ladder.count > 8 || a.ladder.ends[a.ladder.count - 1] != a.hidden)
        throw std::runtime_error("forward: the ladder's widest prefix must equal hidden");
    for (uint32_t band = 0, begin = 0; band < a.ladder.count; begin = a.ladder.ends[band++])
        if (a.ladder.ends[band] % 16 || a.ladder.ends[band] <= begin)
            throw std::runtime_error("forward: band edges must ascend in multiples of 16");
    uint32_t const column_tiles = a.rows_c / fwd_cols;
    if (a.tiles_per_run == 0 || column_tiles % a.tiles_per_run)
        throw std::runtime_error("forward: tiles_per_run must divide the number of candidate tiles");
    if (a.pull.bytes[0] % 16 || a.pull.bytes[1] % 16) throw std::runtime_error("forward: pull sizes must be multiples of 16");
    if (a.multiprocessors < 1) throw std::runtime_error("forward: the multiprocessor count must be positive");

    fwd_params p{};
    p.q_inv = a.query_inverse_norms, p.c_inv = a.candidate_inverse_norms, p.c_tile_max = a.candidate_tile_max;
    p.cube = static_cast<__nv_bfloat16*>(a.gradient_cube_bf16);
    p.partials = a.partials, p.status = a.status;
    p.rows_q = a.rows_q, p.rows_c = a.rows_c, p.hidden = a.hidden;
    p.ladder.count = a.ladder.count;
    for (int i = 0; i < 8; ++i) p.ladder.ends[i] = a.ladder.ends[i];
    p.tiles_per_run = a.tiles_per_run;
    p.runs_per_strip = column_tiles / a.tiles_per_run;
    p.items = (a.rows_q / fwd_rows) * p.runs_per_strip;
    p.beta = a.beta, p.bias = a.bias, p.weight = a.weight;
    p.scalars = a.scalars;
    p.query_base = a.query_base, p.candidate_base = a.candidate_base, p.spec_code = a.spec_code;
    p.budget_ns = a.budget_ns;
    p.pull = a.pull;
    p.trace = a.trace;
    for (uint32_t chunk = 0; chunk < a.hidden / fwd_depth; ++chunk) {
        uint32_t word = 0;
        for (uint32_t sub = 0; sub < 4; ++sub) {
            uint32_t const above = (chunk * 4 + sub + 1) * 16; // first channel above this step
            bool starts = above == a.hidden;
            for (uint32_t band = 0; band + 1 < a.ladder.count; ++band) starts |= a.ladder.ends[band] == above;
            word |= (starts ? 1u : 0u) << (8 * sub);
        }
        p.band_starts[chunk] = word;
    }
    int blocks = static_cast<int>(p.items < static_cast<uint32_t>(a.multiprocessors) ? p.items : a.multiprocessors);
    if ((a.pull.bytes[0] | a.pull.bytes[1]) != 0 && blocks < a.multiprocessors / 2) blocks = a.multiprocessors / 2;
    if (blocks < 1) blocks = 1;

    if (a.fused) {
        if (!forward_fused_supported(a.hidden, a.ladder.count))
            throw std::runtime_error("forward: the fused kernel takes ladders of at most six prefixes");
        if (a.tiles_per_run > fz_max_tiles_per_run) throw std::runtime_error("forward: a fused run holds at most 16 tiles");
        if (a.fused_scratch_bytes < forward_fused_scratch_bytes(a.ladder.count, a.tiles_per_run, blocks))
            throw std::runtime_error("forward: the fused kernel's scratch is too small");
        if (a.fused_scratch_bf16 == nullptr || a.transposed_candidates == nullptr || a.query_gradient == nullptr)
            throw std::runtime_error("forward: the fused kernel needs its scratch, the transposed candidates and the gradient");
    }
    // Everything above is checked before the first driver or runtime call.
    CUtensorMap const& q_map = operand_map(a.queries_bf16, a.hidden, a.rows_q, fwd_depth, fwd_rows);
    CUtensorMap const& c_map = operand_map(a.candidates_bf16, a.hidden, a.rows_c, fwd_depth, fwd_cols);
    fz_maps gemm_maps{};
    if (!a.fused) {
        // The warps' patches of the gradient cube [K, rows_q, rows_c]: boxes of 32 rows x 16 candidates, unswizzled.
        cuuint64_t const dims[3] = {a.rows_c, a.rows_q, a.ladder.count};
        cuuint64_t const strides[2] = {static_cast<cuuint64_t>(a.rows_c) * 2, static_cast<cuuint64_t>(a.rows_c) * a.rows_q * 2};
        cuuint32_t const box[3] = {fwd_chunk_columns, 32, 1};
        CUtensorMap const& cube_map =
            cached_map(a.gradient_cube_bf16, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE);
        launch_for_count<false>(a.ladder.count, q_map, c_map, cube_map, gemm_maps, p, blocks, stream);
    } else {
        p.gradient = a.query_gradient, p.gradient_scale = a.gradient_scale;
        for (uint32_t band = 0, begin = 0; band < a.ladder.count; begin = a.ladder.ends[band++])
            for (uint32_t channel = begin; channel < a.ladder.ends[band]; channel += fz_max_width) {
                if (p.tile_count == fz_max_tiles) throw std::runtime_error("forward: too many channel tiles for the fused kernel");
                uint32_t const left = a.ladder.ends[band] - channel;
                p.tiles[p.tile_count++] = band | ((channel / 16) << 4) | (((left < fz_max_width ? left : fz_max_width) / 16) << 16);
            }
        // Scratch of gradient patches: [CTA and buffer][band][128 rows][run of candidates], written in the warps' boxes
        // (unswizzled), read back as the GEMM's A operand (128 rows x 64 candidates, swizzled).
        uint64_t const run = static_cast<uint64_t>(a.tiles_per_run) * fwd_cols;
        cuuint64_t const dims[3] = {run, fwd_rows, static_cast<cuuint64_t>(blocks) * 2 * a.ladder.count};
        cuuint64_t const strides[2] = {run * 2, run * fwd_rows * 2};
        cuuint32_t const store_box[3] = {fwd_chunk_columns, 32, 1};
        cuuint32_t const load_box[3] = {fz_depth, fwd_rows, 1};
        CUtensorMap const& store_map =
            cached_map(a.fused_scratch_bf16, 3, dims, strides, store_box, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE);
        gemm_maps.patches =
            cached_map(a.fused_scratch_bf16, 3, dims, strides, load_box, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        for (uint32_t index = 0; index < fz_candidate_maps; ++index) {
            // A box may not be taller than the tensor; such a box is never asked for either (tiles are at most `hidden` wide).
            uint32_t const channels = 16u << index;
            gemm_maps.candidates[index] =
                operand_map(a.transposed_candidates, a.rows_c, a.hidden, fz_depth, channels <= a.hidden ? channels : 16u);
        }
        launch_for_count<true>(a.ladder.count, q_map, c_map, store_map, gemm_maps, p, blocks, stream);
    }
    cudaError_t const error = cudaGetLastError();
    if (error != cudaSuccess) throw std::runtime_error(std::string("forward launch failed: ") + cudaGetErrorString(error));
    note_launch();
}

SC_DEFINE_BOUNDS_READER(bounds_record_forward)

void preload_forward_kernels() {
    cudaFuncAttributes attributes;
    require(cudaFuncGetAttributes(&attributes, forward_kernel<1, false>), "preload forward<1>");
    require(cudaFuncGetAttributes(&attributes, forward_kernel<2, false>), "preload forward<2>");
    require(cudaFuncGetAttributes(&attributes, forward_kernel<3, false>), "preload forward<3>");
    require(cudaFuncGetAttributes(&attributes, forward_kernel<4, false>), "preload forward<4>");
    require(cudaFuncGetAttributes(&attributes, forward_kernel<5, false>), "preload forward<5>");
    require(cudaFuncGetAttributes(&attributes, forward_kernel<6, false>), "preload forward<6>");
    require(cudaFuncGetAttributes(&attributes, forward_kernel<7, false>), "preload forward<7>");
    require(cudaFuncGetAttributes(&attributes, forward_kernel<8, false>), "preload forward<8>");
    require(cudaFuncGetAttributes(&attributes, forward_kernel<1, true>), "preload fused forward<1>");
    require(cudaFuncGetAttributes(&attributes, forward_kernel<2, true>), "preload fused forward<2>");
    require(cudaFuncGetAttributes(&attributes, forward_kernel<3, true>), "preload fused forward<3>");
    require(cudaFuncGetAttributes(&attributes, forward_kernel<4, true>), "preload fused forward<4>");
    require(cudaFuncGetAttributes(&attributes, forward_kernel<5, true>), "preload fused forward<5>");
    require(cudaFuncGetAttributes(&attributes, forward_kernel<6, true>), "preload fused forward<6>");
}

} // namespace sc
