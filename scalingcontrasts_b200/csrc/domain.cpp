#include "domain.h"

#include <unistd.h>

#include <algorithm>

#include "driver.h"

namespace sc {

namespace {

CUmemAllocationProp replica_properties(int device) {
    CUmemAllocationProp properties{};
    properties.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    properties.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    properties.location.id = device;
    properties.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return properties;
}

CUmulticastObjectProp multicast_properties(int members, size_t bytes) {
    CUmulticastObjectProp properties{};
    properties.numDevices = static_cast<unsigned int>(members);
    properties.size = bytes;
    properties.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    properties.flags = 0;
    return properties;
}

size_t round_up(size_t value, size_t multiple) { return (value + multiple - 1) / multiple * multiple; }

} // namespace

bool native_domain::multicast_supported(int device) {
    CUdevice handle;
    if (SC_DRIVER_CALL(cuDeviceGet, &handle, device) != CUDA_SUCCESS) return false;
    int supported = 0;
    if (SC_DRIVER_CALL(cuDeviceGetAttribute, &supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, handle) != CUDA_SUCCESS)
        return false;
    return supported != 0;
}

native_domain::native_domain(int device, int member, int members, size_t bytes, bool want_multicast)
    : device_(device), member_(member), members_(members), bytes_(bytes), want_multicast_(want_multicast),
      handles_(members, 0), have_handle_(members, false), mapped_(members, false) {
    if (members < 1 || members > 16 || member < 0 || member >= members) throw std::runtime_error("domain: bad member count");
    require(cudaSetDevice(device), "cudaSetDevice");
    require(cudaFree(nullptr), "context creation");
    CUmemAllocationProp const properties = replica_properties(device);
    size_t granularity = 0;
    SC_DRIVER(cuMemGetAllocationGranularity, &granularity, &properties, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
    if (want_multicast_) {
        if (!multicast_supported(device)) {
            want_multicast_ = false;
        } else {
            CUmulticastObjectProp const multicast = multicast_properties(members, bytes);
            size_t multicast_granularity = 0;
            SC_DRIVER(cuMulticastGetGranularity, &multicast_granularity, &multicast, CU_MULTICAST_GRANULARITY_RECOMMENDED);
            granularity = std::max(granularity, multicast_granularity);
        }
    }
    stride_ = round_up(std::max<size_t>(bytes, 1), granularity);
    SC_DRIVER(cuMemCreate, &handles_[member], stride_, &properties, 0);
    have_handle_[member] = true;
}

native_domain::~native_domain() {
    try {
        close();
    } catch (...) {
    }
}

int native_domain::export_replica() {
    int descriptor = -1;
    SC_DRIVER(cuMemExportToShareableHandle, &descriptor, handles_[member_], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    return descriptor;
}

void native_domain::import_replica(int member, int descriptor) {
    if (member < 0 || member >= members_ || member == member_) throw std::runtime_error("domain: bad peer to import");
    SC_DRIVER(cuMemImportFromShareableHandle, &handles_[member],
              reinterpret_cast<void*>(static_cast<uintptr_t>(descriptor)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    have_handle_[member] = true;
}

int native_domain::create_multicast() {
    if (!want_multicast_) throw std::runtime_error("domain: multicast not available on this device");
    CUmulticastObjectProp const properties = multicast_properties(members_, stride_);
    SC_DRIVER(cuMulticastCreate, &multicast_handle_, &properties);
    have_multicast_handle_ = true;
    int descriptor = -1;
    SC_DRIVER(cuMemExportToShareableHandle, &descriptor, multicast_handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    return descriptor;
}

void native_domain::import_multicast(int descriptor) {
    SC_DRIVER(cuMemImportFromShareableHandle, &multicast_handle_,
              reinterpret_cast<void*>(static_cast<uintptr_t>(descriptor)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    have_multicast_handle_ = true;
}

void native_domain::add_device() {
    if (!have_multicast_handle_) throw std::runtime_error("domain: no multicast object to join");
    CUdevice handle;
    SC_DRIVER(cuDeviceGet, &handle, device_);
    SC_DRIVER(cuMulticastAddDevice, multicast_handle_, handle);
}

void native_domain::map_replicas() {
    for (int m = 0; m < members_; ++m)
        if (!have_handle_[m]) throw std::runtime_error("domain: a peer's replica was never imported");
    SC_DRIVER(cuMemAddressReserve, &replicas_base_, stride_ * members_, 0, 0, 0);
    CUmemAccessDesc access{};
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = device_;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    for (int m = 0; m < members_; ++m) {
        SC_DRIVER(cuMemMap, replicas_base_ + stride_ * m, stride_, 0, handles_[m], 0);
        mapped_[m] = true;
    }
    SC_DRIVER(cuMemSetAccess, replicas_base_, stride_ * members_, &access, 1);
}

void native_domain::bind_multicast() {
    if (!have_multicast_handle_) throw std::runtime_error("domain: no multicast object to bind");
    SC_DRIVER(cuMulticastBindMem, multicast_handle_, 0, handles_[member_], 0, stride_, 0);
    bound_ = true;
    SC_DRIVER(cuMemAddressReserve, &multicast_base_, stride_, 0, 0, 0);
    SC_DRIVER(cuMemMap, multicast_base_, stride_, 0, multicast_handle_, 0);
    multicast_mapped_ = true;
    CUmemAccessDesc access{};
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = device_;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    SC_DRIVER(cuMemSetAccess, multicast_base_, stride_, &access, 1);
}

void native_domain::zero_own() {
    require(cudaSetDevice(device_), "cudaSetDevice");
    require(cudaMemset(reinterpret_cast<void*>(replica(member_)), 0, stride_), "zeroing the replica");
    require(cudaDeviceSynchronize(), "draining after zeroing");
}

void native_domain::close() {
    if (closed_) return;
    closed_ = true;
    cudaSetDevice(device_);
    cudaDeviceSynchronize();
    if (multicast_mapped_) SC_DRIVER_CALL(cuMemUnmap, multicast_base_, stride_);
    if (multicast_base_) SC_DRIVER_CALL(cuMemAddressFree, multicast_base_, stride_);
    if (bound_) {
        CUdevice handle;
        if (SC_DRIVER_CALL(cuDeviceGet, &handle, device_) == CUDA_SUCCESS)
            SC_DRIVER_CALL(cuMulticastUnbind, multicast_handle_, handle, 0, stride_);
    }
    for (int m = 0; m < members_; ++m)
        if (mapped_[m]) SC_DRIVER_CALL(cuMemUnmap, replicas_base_ + stride_ * m, stride_);
    if (replicas_base_) SC_DRIVER_CALL(cuMemAddressFree, replicas_base_, stride_ * members_);
    for (int m = 0; m < members_; ++m)
        if (have_handle_[m]) SC_DRIVER_CALL(cuMemRelease, handles_[m]);
    if (have_multicast_handle_) SC_DRIVER_CALL(cuMemRelease, multicast_handle_);
    multicast_base_ = 0;
    replicas_base_ = 0;
}

} // namespace sc
