// Symmetric memory of one box: every member GPU holds one replica of the same size; each process maps all replicas
// into one contiguous address range (replica m at base + m * stride) and, where the fabric supports it, one multicast
// alias through which `multimem` instructions reach every replica at once.
//
// One process per GPU: physical allocations and the multicast object are shared between processes as POSIX file
// descriptors (the caller moves the descriptors; this class only exports and imports them).
//
// Parity: multimem_domain_t::make and its destructor (scalingcontrasts.cuh:244-410), which builds the same objects
// inside a single process.
#pragma once

#include <cuda.h>

#include <cstddef>
#include <cstdint>
#include <vector>

namespace sc {

class native_domain {
  public:
    native_domain(int device, int member, int members, size_t bytes, bool want_multicast);
    ~native_domain();
    native_domain(native_domain const&) = delete;
    native_domain& operator=(native_domain const&) = delete;

    static bool multicast_supported(int device);

    int export_replica();             // file descriptor of this member's physical allocation (caller closes)
    void import_replica(int member, int descriptor);
    int create_multicast();           // member 0 only: creates the object, returns its descriptor (caller closes)
    void import_multicast(int descriptor);
    void add_device();                // every member, before anyone binds
    void map_replicas();              // after every peer has been imported
    void bind_multicast();            // after every member has added its device
    void zero_own();                  // blocking
    void close();                     // idempotent; the caller makes sure no member still uses the memory

    uint64_t replica(int member) const { return replicas_base_ + static_cast<uint64_t>(member) * stride_; }
    uint64_t multicast() const { return multicast_base_; }
    size_t stride() const { return stride_; }
    size_t bytes() const { return bytes_; }
    int members() const { return members_; }
    int member() const { return member_; }
    int device() const { return device_; }
    bool has_multicast() const { return multicast_base_ != 0; }

  private:
    int device_, member_, members_;
    size_t bytes_, stride_ = 0;
    bool want_multicast_;
    std::vector<CUmemGenericAllocationHandle> handles_;
    std::vector<bool> have_handle_;
    std::vector<bool> mapped_;
    CUmemGenericAllocationHandle multicast_handle_ = 0;
    bool have_multicast_handle_ = false, bound_ = false, multicast_mapped_ = false;
    CUdeviceptr replicas_base_ = 0, multicast_base_ = 0;
    bool closed_ = false;
};

} // namespace sc
