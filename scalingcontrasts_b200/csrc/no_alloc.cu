// The allocation-free backward fold. See no_alloc.h for who needs it and for the contract.
#include "no_alloc.h"

#include <cstdio>
#include <cstring>
#include <mutex>
#include <stdexcept>

#include <cuda_runtime.h>

#include "api.h"

namespace {

// The workspace: the transposed candidates [hidden, rows_c] of one call. In host code this name is only a stand-in for
// the symbol; the device address comes from cudaGetSymbolAddress below, per device.
static __device__ __align__(256) unsigned char workspace[SC_NO_ALLOC_WORKSPACE_BYTES];

constexpr int max_devices = 64;
std::mutex setup_mutex;
void* workspace_address[max_devices] = {};
bool workspace_ready[max_devices] = {};

int fail(int code, char const* message, char* error, size_t capacity) {
    if (error != nullptr && capacity > 0) {
        std::strncpy(error, message, capacity - 1);
        error[capacity - 1] = '\0';
    }
    return code;
}

// Device address of the workspace on the current device, looked up once per device.
int locate_workspace(void** address, char* error, size_t capacity) {
    int device = -1;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess) return fail(SC_NO_ALLOC_CUDA_ERROR, cudaGetErrorString(status), error, capacity);
    if (device < 0 || device >= max_devices) return fail(SC_NO_ALLOC_BAD_ARGUMENT, "device index out of range", error, capacity);
    std::lock_guard<std::mutex> guard(setup_mutex);
    if (!workspace_ready[device]) {
        void* found = nullptr;
        status = cudaGetSymbolAddress(&found, workspace);
        if (status != cudaSuccess || found == nullptr) {
            char message[160];
            std::snprintf(message, sizeof(message), "cudaGetSymbolAddress(workspace) failed on device %d: %s", device,
                          cudaGetErrorString(status));
            return fail(SC_NO_ALLOC_CUDA_ERROR, message, error, capacity);
        }
        workspace_address[device] = found;
        workspace_ready[device] = true;
    }
    *address = workspace_address[device];
    return SC_NO_ALLOC_OK;
}

} // namespace

extern "C" int sc_fold_gradient_no_alloc(const void* cube, const void* candidates, float* query_gradient, uint32_t rows_q,
                                         uint32_t rows_c, uint32_t hidden, const uint32_t* ends, uint32_t prefixes, float scale,
                                         uint32_t* status, void* stream, char* error, size_t error_capacity) {
    if (cube == nullptr || candidates == nullptr || query_gradient == nullptr || ends == nullptr)
        return fail(SC_NO_ALLOC_BAD_ARGUMENT, "cube, candidates, query_gradient and ends must not be null", error, error_capacity);
    if (prefixes < 1 || prefixes > sc::max_prefixes)
        return fail(SC_NO_ALLOC_BAD_ARGUMENT, "a ladder holds 1..8 prefixes", error, error_capacity);
    if (rows_q == 0 || rows_c == 0 || hidden == 0 || rows_q % 128 || rows_c % 64 || hidden % 16 || ends[prefixes - 1] != hidden)
        return fail(SC_NO_ALLOC_BAD_ARGUMENT,
                    "rows_q must be a multiple of 128, rows_c of 64, hidden of 16 and equal to the last prefix end", error,
                    error_capacity);
    // The whole ladder is checked before anything is launched: ends are multiples of 16, strictly ascending, and cut the
    // channels into at most 32 tiles of up to 256 channels (what one backward launch holds).
    uint32_t begin = 0, tiles = 0;
    for (uint32_t band = 0; band < prefixes; ++band) {
        if (ends[band] % 16 || ends[band] <= begin)
            return fail(SC_NO_ALLOC_BAD_ARGUMENT, "prefix ends must ascend strictly in multiples of 16", error, error_capacity);
        tiles += (ends[band] - begin + 255) / 256;
        begin = ends[band];
    }
    if (tiles > 32) return fail(SC_NO_ALLOC_BAD_ARGUMENT, "the ladder cuts the channels into more than 32 tiles", error, error_capacity);
    unsigned long long const needed = 2ull * rows_c * hidden;
    if (needed > SC_NO_ALLOC_WORKSPACE_BYTES) {
        char message[200];
        std::snprintf(message, sizeof(message),
                      "rows_c * hidden * 2 = %llu bytes exceeds the built-in workspace of %u bytes; use the ordinary path with a "
                      "caller-provided buffer",
                      needed, SC_NO_ALLOC_WORKSPACE_BYTES);
        return fail(SC_NO_ALLOC_TOO_LARGE, message, error, error_capacity);
    }
    void* transposed = nullptr;
    int const located = locate_workspace(&transposed, error, error_capacity);
    if (located != SC_NO_ALLOC_OK) return located;
    try {
        cudaStream_t const on = static_cast<cudaStream_t>(stream);
        // Every element of the part of the workspace that the fold reads is written here first.
        sc::launch_transpose(candidates, transposed, rows_c, hidden, on);
        sc::backward_arguments arguments{};
        arguments.gradient_cube_bf16 = cube;
        arguments.transposed_candidates = transposed;
        arguments.query_gradient = query_gradient;
        arguments.status = status;
        arguments.rows_q = rows_q, arguments.rows_c = rows_c, arguments.hidden = hidden;
        arguments.ladder.count = prefixes;
        for (uint32_t band = 0; band < sc::max_prefixes; ++band) arguments.ladder.ends[band] = band < prefixes ? ends[band] : 0;
        arguments.split = 1;
        arguments.scale = scale;
        arguments.budget_ns = 2000000000ull;
        sc::launch_backward(arguments, on);
    } catch (std::exception const& problem) {
        return fail(SC_NO_ALLOC_CUDA_ERROR, problem.what(), error, error_capacity);
    }
    return SC_NO_ALLOC_OK;
}
