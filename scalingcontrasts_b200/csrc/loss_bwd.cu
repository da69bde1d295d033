// Backward tile kernel of the streamed loss: folds a block's per-band gradient cubes into the owner's rows,
//   query_gradient[i, h] += sum_j G_band(h)[i, j] * candidate[j, h],
// as tcgen05 GEMM tiles of 128 rows x up to 256 channels, the candidate index as the K dimension in stages of 64.
// A channel tile never crosses a band edge (edges are multiples of 16 channels and a tile is a multiple of 16 wide),
// so its A operand is a single band's cube, read through a three-dimensional TMA map. The candidates are the B operand
// in one of two layouts: as they are, [R, H] row-major, read in boxes of 64 channels x 64 candidates and handed to the
// tensor cores as an MN-major operand (the channels, the GEMM's N, are the contiguous dimension), which needs no copy of
// the block; or transposed, [H, R], K-major, for callers that hold them that way.
//
// A CTA owns one or two 128-row blocks of a strip and up to 512 tensor-memory columns of accumulators: two blocks x up to
// 256 channels (both blocks use the same candidate stage, which halves the candidate refills from L2), or, for a band of
// 257 to 384 channels, one block x the whole band, so that the band's cube, the traffic this kernel is bound by, is read
// from DRAM once instead of once per 256-channel tile.
//
// Warp roles (192 threads): warps 0-3 epilogue (tensor-memory lanes 32*w..), warp 4 TMA producer, warp 5 UMMA issuer
// and tensor-memory owner. The producer and the issuer run warp-wide with only the TMA / UMMA / commit instructions
// under the elected lane, so that their operands are warp-uniform values. The epilogue adds its scaled accumulators with
// vector reductions (fire and forget: no read of the old value comes back to the SM). With `split == 1` each output
// element receives exactly one addition per launch, so the sum's order is the launches' stream order and the result
// is deterministic; with a larger split the candidate range is divided and the order of a launch's partial sums is not.
//
// Parity: backward_tile_cuda_ (scalingcontrasts.cuh:1042-1136).
#include <array>
#include <stdexcept>
#include <string>
#include <vector>

#include "api.h"
#include "common.cuh"
#include "driver.h"

namespace sc {

namespace {

constexpr uint32_t bwd_rows = 128;
constexpr uint32_t bwd_depth = 64;        // candidates per stage
constexpr uint32_t bwd_max_width = 256;   // channels per UMMA and per tile of a two-block CTA
constexpr uint32_t bwd_wide_width = 384;  // channels of a one-block CTA that takes a whole band
constexpr uint32_t bwd_stages = 6;                                  // at most
constexpr uint32_t bwd_a_bytes = bwd_rows * bwd_depth * 2;        // one 128-row block of the cube
constexpr uint32_t bwd_b_bytes = bwd_max_width * bwd_depth * 2;
constexpr uint32_t bwd_stage_bytes = 2 * bwd_a_bytes + bwd_b_bytes; // two row blocks share one candidate tile
static_assert(bwd_a_bytes + bwd_wide_width * bwd_depth * 2 <= bwd_stage_bytes, "a wide one-block stage must fit a stage");
constexpr uint32_t bwd_tmem_columns = 512;
constexpr uint32_t bwd_block_columns = 256;                         // tensor-memory columns between the two accumulators
constexpr uint32_t bwd_threads = 192;
constexpr uint32_t bwd_max_tiles = 32;

struct bwd_tail {
    uint64_t stage_full[bwd_stages];
    uint64_t stage_empty[bwd_stages];
    uint64_t accumulated;
    uint32_t tmem_base;
    uint32_t abort_flag;
};
// The ring of stages: 208 KB; a stage is the CTA's row blocks of the cube plus the candidates of the tile's own width.
constexpr uint32_t bwd_ring_bytes = 208 * 1024;
constexpr uint32_t bwd_shared_bytes = 1024 + bwd_ring_bytes + sizeof(bwd_tail);
static_assert(3 * bwd_stage_bytes <= bwd_ring_bytes, "three of the largest stages must fit the ring");
static_assert(bwd_shared_bytes <= 227 * 1024, "the kernel's shared memory must fit one CTA's maximum");
constexpr uint32_t bwd_candidate_maps = 5;                          // boxes of 16, 32, 64, 128 and 256 channels

struct bwd_tile {
    uint32_t band, channel0, width;
    uint32_t blocks;    // row blocks per CTA of this tile: 1 or 2
    uint32_t first_cta; // first CTA of the tile's group; a group's CTAs walk its tiles fastest, then the row blocks
    uint32_t group;     // tiles in the group: the tiles of one band (they read the same rows of the cube)
};

// The transposed candidates under five tensor maps that differ only in the box's channel count (16 << index): a tile's
// channels are fetched greedily with the largest boxes that fit, so a stage takes one to three candidate loads.
struct bwd_candidate_boxes {
    CUtensorMap maps[bwd_candidate_maps];
};


struct bwd_params {
    float* query_gradient;
    uint32_t* status;
    uint32_t rows_q, rows_c, hidden;
    uint32_t tile_count, split;
    float scale; // applied to every product before it is added: the loss's 2/N (mirror cell and weight)
    uint64_t budget_ns;
    bwd_tile tiles[bwd_max_tiles];
};

// Shared-memory descriptor words of the B operand. K-major (transposed candidates): rows of 64 candidates, eight rows
// per 1024-byte swizzle atom, atoms 1024 bytes apart along N; a step of 16 candidates adds 32 bytes. MN-major (row-major
// candidates): a box is 64 candidates (K) x 64 channels (N, contiguous, one 128-byte row per candidate); eight
// candidates make one atom, atoms follow each other every 1024 bytes along K (the stride offset), boxes of 64 channels
// every 8192 bytes along N (the leading offset); a step of 16 candidates is two atoms, 2048 bytes.
constexpr uint32_t bwd_mn_box_bytes = 64 * bwd_depth * 2;

template <bool mn_major_>
__global__ void __launch_bounds__(bwd_threads, 1)
    backward_kernel(const __grid_constant__ CUtensorMap cube_map, const __grid_constant__ bwd_candidate_boxes candidates,
                    const bwd_params p) {
    extern __shared__ uint8_t raw_shared[];
    uint32_t const raw_address = smem_u32(raw_shared);
    uint32_t const stages_base = (raw_address + 1023u) & ~1023u;
    bwd_tail* tail = reinterpret_cast<bwd_tail*>(raw_shared + (stages_base - raw_address) + bwd_ring_bytes);
    uint32_t const warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    uint32_t tile_index = 0; // the first tile of the group this CTA falls into, then the CTA's own tile within it
    while (tile_index + p.tiles[tile_index].group < p.tile_count &&
           blockIdx.x >= p.tiles[tile_index + p.tiles[tile_index].group].first_cta)
        tile_index += p.tiles[tile_index].group;
    uint32_t const within = blockIdx.x - p.tiles[tile_index].first_cta, group = p.tiles[tile_index].group;
    tile_index += within % group;
    bwd_tile const tile = p.tiles[tile_index];
    // Stage geometry: [row blocks of the cube, 16 KB each][candidate tile of the tile's width]. MN-major candidates come in
    // whole boxes of 64 channels (8 KB), K-major ones in rows of 128 bytes per channel; either way a stage is a multiple of
    // 1 KB, so every stage starts on a swizzle atom.
    bool const wide = tile.width > bwd_max_width;
    uint32_t const candidate_bytes = mn_major_ ? ((tile.width + 63u) / 64u) * bwd_mn_box_bytes : tile.width * bwd_depth * 2u;
    uint32_t const stage_bytes = tile.blocks * bwd_a_bytes + candidate_bytes;
    // One-block tiles (small launches) take as deep a ring as fits: 0.187 -> 0.181 ms per 4096-row block. Two-block tiles
    // stay at three stages: deeper rings for the narrow, DRAM-bound ones made a 16384-row launch slower (1.82 -> 1.85 ms per
    // block), their CTAs then take bandwidth from the wide ones that finish last.
    uint32_t const stages = tile.blocks == 2 ? 3u : min(bwd_stages, bwd_ring_bytes / stage_bytes);
    uint32_t const b_offset = tile.blocks * bwd_a_bytes;
    uint32_t const first_block = within / group * tile.blocks;
    uint32_t const blocks = min(tile.blocks, p.rows_q / bwd_rows - first_block);
    uint32_t const chunks_total = p.rows_c / bwd_depth;
    uint32_t const chunks_per_split = (chunks_total + p.split - 1) / p.split;
    uint32_t const chunk_begin = min(blockIdx.y * chunks_per_split, chunks_total);
    uint32_t const chunk_end = min(chunk_begin + chunks_per_split, chunks_total);

    if (threadIdx.x == 0) {
        tail->abort_flag = status_poisoned(p.status) ? 1u : 0u;
        for (uint32_t i = 0; i < bwd_stages; ++i) {
            mbar_init(smem_u32(&tail->stage_full[i]), 1);
            mbar_init(smem_u32(&tail->stage_empty[i]), 1);
        }
        mbar_init(smem_u32(&tail->accumulated), 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (tail->abort_flag != 0u || chunk_begin >= chunk_end) return;
    if (warp == 5) {
        tmem_alloc(smem_u32(&tail->tmem_base), bwd_tmem_columns);
        tmem_relinquish();
    }
    if (warp == 4 && lane == 0) {
        tma_prefetch_descriptor(&cube_map);
        for (uint32_t i = 0; i < bwd_candidate_maps; ++i) tma_prefetch_descriptor(&candidates.maps[i]);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    uint32_t const tmem_base = tail->tmem_base;
    wait_context const ctx{p.status, p.budget_ns, &tail->abort_flag};

    if (warp == 4) {
        bool const elected = elect_one();
        uint32_t stage = 0, phase = 0;
        uint32_t const boxes = (tile.width + 63u) / 64u; // MN-major: whole boxes of 64 channels, the last one partly used
        uint32_t const bytes = blocks * bwd_a_bytes + (mn_major_ ? boxes * bwd_mn_box_bytes : tile.width * bwd_depth * 2);
        for (uint32_t chunk = chunk_begin; chunk < chunk_end; ++chunk) {
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&tail->stage_empty[stage]), phase ^ 1u, ctx, site_bwd_stage_empty, chunk)))
                break;
            uint32_t const full = smem_u32(&tail->stage_full[stage]);
            uint32_t const destination = stages_base + stage * stage_bytes;
            if (elected) {
                mbar_arrive_expect_tx(full, bytes);
                for (uint32_t block = 0; block < blocks; ++block)
                    tma_load_3d(destination + block * bwd_a_bytes, &cube_map, full, static_cast<int>(chunk * bwd_depth),
                                static_cast<int>((first_block + block) * bwd_rows), static_cast<int>(tile.band));
                if constexpr (mn_major_) {
                    // Boxes of 64 channels x 64 candidates straight from the row-major block; channels past the tile (or
                    // past the tensor, which the load fills with zeros) are carried along and never multiplied.
                    for (uint32_t box = 0; box < boxes; ++box)
                        tma_load_2d(destination + b_offset + box * bwd_mn_box_bytes, &candidates.maps[0], full,
                                    static_cast<int>(tile.channel0 + box * 64u), static_cast<int>(chunk * bwd_depth));
                } else {
                    // Largest boxes first; 16 channels are 2048 bytes of the stage (rows of 128 bytes under the swizzle).
                    uint32_t done = 0;
#pragma unroll
                    for (int index = static_cast<int>(bwd_candidate_maps) - 1; index >= 0; --index) {
                        uint32_t const box = 16u << index;
                        if (tile.width - done >= box) {
                            tma_load_2d(destination + b_offset + done * 128u, &candidates.maps[index], full,
                                        static_cast<int>(chunk * bwd_depth), static_cast<int>(tile.channel0 + done));
                            done += box;
                        }
                    }
                }
            }
            __syncwarp();
            if (++stage == stages) stage = 0, phase ^= 1u;
        }
    } else if (warp == 5) {
        bool const elected = elect_one();
        // A tile wider than one UMMA's 256 columns is issued in two pieces; the second starts 256 channels on, which is
        // 32 KB into the candidate stage in either layout (four 8 KB boxes, or 256 rows of 128 bytes).
        uint32_t const major = mn_major_ ? umma_idesc_b_mn_major : 0u;
        uint32_t const width0 = wide ? bwd_max_width : tile.width;
        uint32_t const idesc0 = umma_idesc_bf16(bwd_rows, width0) | major;
        uint32_t const idesc1 = wide ? (umma_idesc_bf16(bwd_rows, tile.width - bwd_max_width) | major) : 0u;
        constexpr uint32_t descriptor_high = (1024u >> 4) | (1u << 14) | (2u << 29); // stride 1024 B, version 1, 128-byte swizzle
        uint32_t const low_base = ((stages_base & 0x3FFFFu) >> 4) | (1u << 16);
        // The B operand's leading offset (bits 16-29 of the low word) and its advance per 16 candidates.
        constexpr uint32_t b_leading = mn_major_ ? ((bwd_mn_box_bytes >> 4) << 16) : (1u << 16);
        constexpr uint32_t b_step = mn_major_ ? (2048u >> 4) : 2u;
        uint32_t stage = 0, phase = 0, accumulate = 0;
        bool ok = true;
        for (uint32_t chunk = chunk_begin; chunk < chunk_end; ++chunk) {
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&tail->stage_full[stage]), phase, ctx, site_bwd_stage_full, chunk));
            if (!ok) break;
            tcgen05_fence_after();
            uint32_t const a_low = low_base + ((stage * stage_bytes) >> 4);
            uint32_t const b_low = (a_low & 0xFFFFu) + (b_offset >> 4) + b_leading;
            for (uint32_t block = 0; block < blocks; ++block) {
#pragma unroll
                for (uint32_t step = 0; step < bwd_depth / 16; ++step) {
                    uint64_t a_descriptor, b_descriptor;
                    asm("mov.b64 %0, {%1, %2};" : "=l"(a_descriptor) : "r"(a_low + block * (bwd_a_bytes >> 4) + step * 2u), "r"(descriptor_high));
                    asm("mov.b64 %0, {%1, %2};" : "=l"(b_descriptor) : "r"(b_low + step * b_step), "r"(descriptor_high));
                    if (elected) {
                        umma_bf16(tmem_base + block * bwd_block_columns, a_descriptor, b_descriptor, idesc0,
                                  step == 0 ? accumulate : 1u);
                        if (wide)
                            umma_bf16(tmem_base + bwd_max_width, a_descriptor, b_descriptor + ((bwd_max_width * bwd_depth * 2u) >> 4),
                                      idesc1, step == 0 ? accumulate : 1u);
                    }
                }
            }
            accumulate = 1;
            if (elected) umma_commit(smem_u32(&tail->stage_empty[stage]));
            __syncwarp();
            if (++stage == stages) stage = 0, phase ^= 1u;
        }
        if (ok && elected) umma_commit(smem_u32(&tail->accumulated));
        __syncwarp();
    } else {
        if (mbar_wait(smem_u32(&tail->accumulated), 0u, ctx, site_bwd_accumulated, tile_index)) {
            tcgen05_fence_after();
          for (uint32_t block = 0; block < blocks; ++block) {
            uint32_t const row = (first_block + block) * bwd_rows + warp * 32 + lane;
            float* destination = p.query_gradient + static_cast<size_t>(row) * p.hidden + tile.channel0;
            uint32_t const lane_base = tmem_base + ((warp * 32u) << 16) + block * bwd_block_columns;
            for (uint32_t column = 0; column < tile.width; column += 16) {
                if (!SC_WARP_IN_BOUNDS(static_cast<size_t>(row) * p.hidden + tile.channel0 + column + 15,
                                       static_cast<size_t>(p.rows_q) * p.hidden))
                    break;
                uint32_t values[16];
                tmem_load_16(lane_base + column, values);
                tmem_load_wait();
#pragma unroll
                for (int v = 0; v < 4; ++v)
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(destination + column + 4 * v),
                                 "f"(p.scale * __uint_as_float(values[4 * v])), "f"(p.scale * __uint_as_float(values[4 * v + 1])),
                                 "f"(p.scale * __uint_as_float(values[4 * v + 2])), "f"(p.scale * __uint_as_float(values[4 * v + 3]))
                                 : "memory");
            }
          }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (tail->abort_flag != 0u) {
        uint64_t const start = global_timer_ns();
        while (global_timer_ns() - start < 200000ull) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 5) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, bwd_tmem_columns);
    }
}

// The launch's tile table: which (band, channels, row blocks per CTA) tiles there are and which CTAs of the
// one-dimensional grid belong to each. Pure arithmetic on the shape, so that it can be checked without a GPU.
uint32_t plan_tiles(uint32_t rows_q, ladder_host const& ladder, uint32_t split, int multiprocessors, bwd_tile* tiles,
                    uint32_t& tile_count) {
    tile_count = 0;
    // Two row blocks per CTA once that still leaves at least two CTAs per multiprocessor with tiles of 256 channels. Only
    // then (a launch bound by the cube's bytes, not by its tail) does a band of 257..384 channels go to one-block CTAs
    // that take it whole; a small launch prefers more and shorter CTAs.
    uint32_t const row_blocks = rows_q / bwd_rows;
    uint32_t plain_tiles = 0, begin = 0;
    for (uint32_t band = 0; band < ladder.count; ++band) {
        uint32_t const end = ladder.ends[band];
        if (end % 16 || end <= begin) throw std::runtime_error("backward: band edges must ascend in multiples of 16");
        plain_tiles += (end - begin + bwd_max_width - 1) / bwd_max_width;
        begin = end;
    }
    bool const two_blocks = static_cast<uint64_t>(row_blocks / 2) * plain_tiles * split >= 2ull * static_cast<uint64_t>(multiprocessors);
    begin = 0;
    for (uint32_t band = 0; band < ladder.count; ++band) {
        uint32_t const end = ladder.ends[band];
        for (uint32_t channel = begin; channel < end;) {
            if (tile_count == bwd_max_tiles) throw std::runtime_error("backward: too many channel tiles for one launch");
            uint32_t const left = end - channel;
            bool const whole_band = two_blocks && left == end - begin && left > bwd_max_width && left <= bwd_wide_width;
            uint32_t const width = whole_band || left <= bwd_max_width ? left : bwd_max_width;
            tiles[tile_count++] = bwd_tile{band, channel, width, two_blocks && !whole_band ? 2u : 1u, 0u, 1u};
            channel += width;
        }
        begin = end;
    }
    // CTAs go band by band in the order the hardware hands them out: two-block tiles before one-block tiles and wider
    // bands before narrower. In a large launch the two-block CTAs of the narrow bands wait for DRAM
    // while the one-block CTAs of a whole wide band are busy with their UMMAs; measured, the launch is fastest with the
    // latter last (1.832 ms per 16384-row block against 1.861 with them first and 1.860 with both kinds mixed pair of
    // row blocks by pair).
    auto band_width = [&](uint32_t band) { return ladder.ends[band] - (band ? ladder.ends[band - 1] : 0u); };
    auto before = [&](bwd_tile const& x, bwd_tile const& y) { // does x go ahead of y?
        if (x.blocks != y.blocks) return x.blocks > y.blocks;
        if (x.band != y.band) return band_width(x.band) != band_width(y.band) ? band_width(x.band) > band_width(y.band) : x.band > y.band;
        return x.width > y.width;
    };
    for (uint32_t i = 1; i < tile_count; ++i)
        for (uint32_t j = i; j > 0 && before(tiles[j], tiles[j - 1]); --j) {
            bwd_tile const held = tiles[j - 1];
            tiles[j - 1] = tiles[j], tiles[j] = held;
        }
    // The tiles of one band read the same rows of the cube. Their CTAs for a row block are handed out one after the
    // other, so that they run side by side at the pace of the slower one and the second read of a row is served by L2.
    uint32_t ctas = 0;
    for (uint32_t i = 0; i < tile_count;) {
        uint32_t members = 1;
        while (i + members < tile_count && tiles[i + members].band == tiles[i].band &&
               tiles[i + members].blocks == tiles[i].blocks)
            ++members;
        for (uint32_t m = 0; m < members; ++m) tiles[i + m].first_cta = ctas, tiles[i + m].group = members;
        ctas += members * ((row_blocks + tiles[i].blocks - 1) / tiles[i].blocks);
        i += members;
    }
    return ctas;
}

} // namespace

void launch_backward(backward_arguments const& a, cudaStream_t stream) {
    if (a.rows_q % bwd_rows || a.rows_c % bwd_depth || a.hidden % 16)
        throw std::runtime_error("backward: rows must be multiples of 128 (queries) and 64 (candidates)");
    if (a.split < 1) throw std::runtime_error("backward: split must be at least 1");
    bwd_params p{};
    p.query_gradient = a.query_gradient, p.status = a.status;
    p.rows_q = a.rows_q, p.rows_c = a.rows_c, p.hidden = a.hidden;
    p.split = a.split, p.budget_ns = a.budget_ns, p.scale = a.scale;
    // Per device, once: the multiprocessor count (a runtime query that needs no context of its own).
    static int counted_device = -1, multiprocessors = 148;
    int device = 0;
    cudaGetDevice(&device);
    if (counted_device != device) {
        if (cudaDeviceGetAttribute(&multiprocessors, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) multiprocessors = 148;
        counted_device = device;
    }
    uint32_t const ctas = plan_tiles(a.rows_q, a.ladder, a.split, multiprocessors, p.tiles, p.tile_count);
    bool const mn_major = a.candidates_row_major != nullptr && a.hidden >= 64;
    if (!mn_major && a.transposed_candidates == nullptr) throw std::runtime_error("backward: no candidates given");
    // Everything above is checked before the first driver or runtime call.
    cuuint64_t const cube_dims[3] = {a.rows_c, a.rows_q, a.ladder.count};
    cuuint64_t const cube_strides[2] = {static_cast<cuuint64_t>(a.rows_c) * 2, static_cast<cuuint64_t>(a.rows_c) * a.rows_q * 2};
    cuuint32_t const cube_box[3] = {bwd_depth, bwd_rows, 1};
    CUtensorMap const& cube_map = cached_map(a.gradient_cube_bf16, 3, cube_dims, cube_strides, cube_box, CU_TENSOR_MAP_SWIZZLE_128B,
                                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    bwd_candidate_boxes candidates;
    for (uint32_t index = 0; index < bwd_candidate_maps; ++index) {
        if (mn_major) {
            // One map over the block as it lies in memory: boxes of 64 channels (the contiguous dimension) x 64 candidates.
            candidates.maps[index] = cached_operand_map(a.candidates_row_major, a.hidden, a.rows_c, 64, bwd_depth);
            continue;
        }
        // A box may not be taller than the tensor; such a box is never asked for either (tiles are at most `hidden` wide).
        uint32_t const channels = 16u << index;
        candidates.maps[index] =
            cached_operand_map(a.transposed_candidates, a.rows_c, a.hidden, bwd_depth, channels <= a.hidden ? channels : 16u);
    }

    // Per device, once: the shared-memory limit of the kernel.
    static int prepared_device = -1;
    if (prepared_device != device) {
        require(cudaFuncSetAttribute(backward_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bwd_shared_bytes),
                "raising the backward kernel's shared memory");
        require(cudaFuncSetAttribute(backward_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bwd_shared_bytes),
                "raising the backward kernel's shared memory");
        prepared_device = device;
    }
    dim3 const grid(ctas, a.split, 1);
    if (mn_major) backward_kernel<true><<<grid, bwd_threads, bwd_shared_bytes, stream>>>(cube_map, candidates, p);
    else backward_kernel<false><<<grid, bwd_threads, bwd_shared_bytes, stream>>>(cube_map, candidates, p);
    cudaError_t const error = cudaGetLastError();
    if (error != cudaSuccess) throw std::runtime_error(std::string("backward launch failed: ") + cudaGetErrorString(error));
    note_launch();
}

void preload_forward_kernels();
std::vector<std::array<uint32_t, 6>> backward_plan(uint32_t rows_q, ladder_host const& ladder, uint32_t split,
                                                    int multiprocessors, uint32_t* ctas) {
    if (rows_q % bwd_rows || split < 1) throw std::runtime_error("backward_plan: rows must be a multiple of 128 and split positive");
    bwd_tile tiles[bwd_max_tiles];
    uint32_t count = 0;
    uint32_t const total = plan_tiles(rows_q, ladder, split, multiprocessors, tiles, count);
    if (ctas) *ctas = total;
    std::vector<std::array<uint32_t, 6>> out;
    for (uint32_t i = 0; i < count; ++i)
        out.push_back({tiles[i].band, tiles[i].channel0, tiles[i].width, tiles[i].blocks, tiles[i].first_cta, tiles[i].group});
    return out;
}

SC_DEFINE_BOUNDS_READER(bounds_record_backward)

void preload_loss_kernels() {
    cudaFuncAttributes attributes;
    require(cudaFuncGetAttributes(&attributes, backward_kernel<false>), "preload backward");
    require(cudaFuncGetAttributes(&attributes, backward_kernel<true>), "preload backward (row-major candidates)");
    preload_forward_kernels();
}

} // namespace sc
