// Driver API entry points resolved at run time through the CUDA runtime, so that the extension does not link libcuda
// and can be imported (and its host-only parts used) on a machine without a driver.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <map>
#include <mutex>
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

// Tiled tensor maps over bfloat16 tensors of up to three dimensions. A map is a pure function of (address, shape, box,
// swizzle, promotion), and a training loop asks for the same few over and over, so encoded maps are kept: a launch costs
// a lookup instead of a driver call per map. Dimensions and strides are innermost first; strides in bytes.
struct tensor_map_key {
    uint64_t words[11];
    bool operator<(tensor_map_key const& other) const {
        for (int i = 0; i < 11; ++i)
            if (words[i] != other.words[i]) return words[i] < other.words[i];
        return false;
    }
};
inline CUtensorMap const& cached_map(void const* base, uint32_t rank, cuuint64_t const (&dims)[3], cuuint64_t const (&strides)[2],
                                     cuuint32_t const (&box)[3], CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promotion) {
    static std::mutex guard;
    static std::map<tensor_map_key, CUtensorMap> maps;
    tensor_map_key const key{{reinterpret_cast<uint64_t>(base), rank, dims[0], dims[1], dims[2], strides[0], strides[1],
                              (static_cast<uint64_t>(box[0]) << 32) | box[1], box[2], static_cast<uint64_t>(swizzle),
                              static_cast<uint64_t>(promotion)}};
    std::lock_guard<std::mutex> const lock(guard);
    auto const found = maps.find(key);
    if (found != maps.end()) return found->second;
    if (maps.size() >= 4096) maps.clear();
    CUtensorMap map;
    cuuint32_t const element_strides[3] = {1, 1, 1};
    SC_DRIVER(cuTensorMapEncodeTiled, &map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box,
              element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promotion, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return maps.emplace(key, map).first->second;
}
// Rows of `inner` bfloat16 values, `outer` of them, read in boxes under the 128-byte swizzle (a UMMA operand).
inline CUtensorMap const& cached_operand_map(void const* base, uint64_t inner, uint64_t outer, uint32_t box_inner,
                                             uint32_t box_outer) {
    cuuint64_t const dims[3] = {inner, outer, 1};
    cuuint64_t const strides[2] = {inner * 2, 0};
    cuuint32_t const box[3] = {box_inner, box_outer, 1};
    return cached_map(base, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
}

} // namespace sc
