// Driver API entry points resolved at run time through the CUDA runtime, so that the extension does not link libcuda
// and can be imported (and its host-only parts used) on a machine without a driver.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

namespace sc {

inline void* resolve_driver(char const* name) {
    void* function = nullptr;
    cudaDriverEntryPointQueryResult result;
    cudaError_t const error = cudaGetDriverEntryPoint(name, &function, cudaEnableDefault, &result);
    if (error != cudaSuccess || function == nullptr || result != cudaDriverEntryPointSuccess)
        throw std::runtime_error(std::string("driver entry point unavailable: ") + name);
    return function;
}

inline std::string driver_error_name(CUresult result);

// Calls driver function `name` with the given arguments; the pointer is looked up once.
#define SC_DRIVER_CALL(name, ...)                                                                                       \
    ([&]() -> CUresult {                                                                                                \
        static auto const function = reinterpret_cast<decltype(&name)>(::sc::resolve_driver(#name));                    \
        return function(__VA_ARGS__);                                                                                   \
    }())

inline std::string driver_error_name(CUresult result) {
    char const* name = nullptr;
    if (SC_DRIVER_CALL(cuGetErrorName, result, &name) != CUDA_SUCCESS || name == nullptr) return "unnamed driver error";
    return name;
}

inline void require(CUresult result, char const* what) {
    if (result != CUDA_SUCCESS) throw std::runtime_error(std::string(what) + " failed: " + driver_error_name(result));
}
inline void require(cudaError_t result, char const* what) {
    if (result != cudaSuccess) throw std::runtime_error(std::string(what) + " failed: " + cudaGetErrorString(result));
}

#define SC_DRIVER(name, ...) ::sc::require(SC_DRIVER_CALL(name, __VA_ARGS__), #name)

} // namespace sc
