// sc_fold_gradient_no_alloc: the backward fold of the streamed loss for callers that must not allocate.
//
// This entry point has no counterpart in the reference. It exists for hosts of this library that cannot obtain device
// memory at the moment they need the result: code that runs inside someone else's memory budget (a plugin or an
// inference server whose pool is fully committed), code on a path where an allocation call is forbidden or unsafe
// (real-time loops, a device whose memory is exhausted by the model itself), and callers that simply have no allocator
// to hand a workspace from. The ordinary path (transpose the candidates into a caller-provided buffer, then run the
// backward tile kernel) needs a workspace of hidden x rows_c bfloat16 values; here that workspace is a fixed array
// inside the library.
//
//   query_gradient[i, h] += scale * sum_j cube[band(h), i, j] * candidates[j, h]
//
// Contract
//   * Nothing is allocated or freed, by this function or by anything it calls: the workspace is a file-scope device
//     array of SC_NO_ALLOC_WORKSPACE_BYTES that every GPU using the library holds from module load until exit.
//   * Limit: rows_c * hidden * 2 bytes must not exceed SC_NO_ALLOC_WORKSPACE_BYTES (for example 1024 candidates of
//     1024 channels, or 2048 of 512). Larger problems are refused with SC_NO_ALLOC_TOO_LARGE and a message; use the
//     ordinary path for them.
//   * The first call on each device looks up the array's device address (with that device current) and keeps it. Make
//     that first call outside of any stream capture. The kept address belongs to the device's current context: after a
//     cudaDeviceReset() it is stale, and this entry point must not be called again in that process.
//   * All calls on a device share the one workspace, and it keeps whatever the previous call left there. Nothing in it
//     has to start at zero: each call overwrites the part it reads before reading it. Two calls whose kernels can run
//     at the same time on one GPU (different streams, no ordering between them) race on the workspace; order them.
//   * Inputs and outputs are the caller's: `cube` is [prefixes, rows_q, rows_c] bfloat16, `candidates` is
//     [rows_c, hidden] bfloat16, `query_gradient` is [rows_q, hidden] float32 and is accumulated into. These three must
//     be 16-byte aligned device pointers on the current device. `ends` is a HOST array of `prefixes` values (it is read
//     on the host, before anything is launched): strictly ascending multiples of 16, the last equal to hidden, cutting
//     the channels into at most 32 tiles of up to 256. rows_q must be a multiple of 128, rows_c of 64. Anything else is
//     refused with SC_NO_ALLOC_BAD_ARGUMENT before any kernel runs or the workspace is touched. `status` may be null; when given it is the eight-word status block of the tile
//     kernels (a bounded wait that runs out is recorded there). `stream` is a cudaStream_t.
//   * Returns SC_NO_ALLOC_OK, or an error code with a zero-terminated message in `error` (when `error` is not null).
#pragma once

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SC_NO_ALLOC_WORKSPACE_BYTES (2u * 1024u * 1024u)

enum {
    SC_NO_ALLOC_OK = 0,
    SC_NO_ALLOC_TOO_LARGE = 1,
    SC_NO_ALLOC_BAD_ARGUMENT = 2,
    SC_NO_ALLOC_CUDA_ERROR = 3,
};

__attribute__((visibility("default"))) int sc_fold_gradient_no_alloc(
    const void* cube, const void* candidates, float* query_gradient, uint32_t rows_q, uint32_t rows_c, uint32_t hidden,
    const uint32_t* ends, uint32_t prefixes, float scale, uint32_t* status, void* stream, char* error, size_t error_capacity);

#ifdef __cplusplus
}
#endif
