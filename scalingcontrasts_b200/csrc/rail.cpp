// The cross-box rail and its loopback transport.
//
// A rail connects one GPU of this host with the same-numbered GPU of another host. It keeps the reference's verbs
// semantics: the embeddings block is written into the peer's landing buffer of the given parity and the peer sees a
// completion carrying the byte count as immediate data; a row of loss summands is written into the peer's
// host-side table the same way; `await_landed` consumes one completion.
//
// This box has one host and no RDMA NIC, so the transport here is a loopback: the "write" is a device-to-device copy
// into memory the peer exported (a CUDA IPC handle across processes, the plain address inside one process), the
// completion queue and the summands table live in a POSIX shared-memory segment owned by the receiver, and the
// completion is pushed by a host callback that the copy's stream runs after the copy. Everything above the transport
// (endpoint exchange, parity double buffering, ordering of await against reads) is what a verbs transport would see.
// Completion errors can be injected from the host to exercise the error path; nothing here can fault a GPU.
//
// Parity: rdma_rail_t / rdma_endpoint_t (scalingcontrasts.cuh:419-646).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstring>
#include <stdexcept>
#include <string>
#include <thread>

#include <cuda_runtime.h>

#include "driver.h"
#include "rail.h"

namespace sc {

namespace {

void check(cudaError_t error, char const* what) {
    if (error != cudaSuccess) throw std::runtime_error(std::string(what) + " failed: " + cudaGetErrorString(error));
}

struct pending_completion {
    rail_mailbox* mailbox;
    uint32_t immediate;
    uint32_t status;
};

void push_completion(rail_mailbox* mailbox, uint32_t immediate, uint32_t status) {
    uint64_t const slot = mailbox->head.fetch_add(1, std::memory_order_acq_rel);
    rail_completion& entry = mailbox->entries[slot % rail_queue_depth];
    entry.immediate = immediate;
    entry.status = status;
    entry.sequence.store(slot + 1, std::memory_order_release);
}

// Base address of the allocation that contains `address` (an IPC handle maps the allocation from its base).
bool allocation_base(uint64_t address, uint64_t* base) {
    CUdeviceptr found = 0;
    size_t size = 0;
    if (SC_DRIVER_CALL(cuMemGetAddressRange, &found, &size, static_cast<CUdeviceptr>(address)) != CUDA_SUCCESS) return false;
    *base = static_cast<uint64_t>(found);
    return true;
}

void CUDART_CB completion_callback(void* data) {
    auto* pending = static_cast<pending_completion*>(data);
    push_completion(pending->mailbox, pending->immediate, pending->status);
    delete pending;
}

} // namespace

loopback_rail::loopback_rail(int device, uint64_t embeddings, uint64_t block_bytes, uint64_t landing, int hosts, int host,
                             std::string const& mailbox_name, uint32_t packet_sequence)
    : device_(device), embeddings_(embeddings), block_bytes_(block_bytes), landing_(landing), hosts_(hosts), host_(host),
      mailbox_name_(mailbox_name) {
    if (hosts < 1 || hosts > rail_max_hosts || host < 0 || host >= hosts) throw std::runtime_error("rail: bad host index");
    check(cudaSetDevice(device), "cudaSetDevice");
    check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "creating the rail's stream");
    // The receiver owns its mailbox: completion queue + summands table.
    int const descriptor = shm_open(mailbox_name.c_str(), O_CREAT | O_RDWR, 0600);
    if (descriptor < 0) throw std::runtime_error("rail: shm_open failed for " + mailbox_name);
    if (ftruncate(descriptor, sizeof(rail_mailbox)) != 0) {
        ::close(descriptor);
        throw std::runtime_error("rail: ftruncate failed for " + mailbox_name);
    }
    void* mapping = mmap(nullptr, sizeof(rail_mailbox), PROT_READ | PROT_WRITE, MAP_SHARED, descriptor, 0);
    ::close(descriptor);
    if (mapping == MAP_FAILED) throw std::runtime_error("rail: mmap failed for " + mailbox_name);
    own_mailbox_ = new (mapping) rail_mailbox();
    own_mailbox_->head.store(0);
    for (auto& entry : own_mailbox_->entries) entry.sequence.store(0);
    std::memset(own_mailbox_->summands, 0, sizeof(own_mailbox_->summands));

    std::memset(&local_, 0, sizeof(local_));
    local_.process = static_cast<uint64_t>(getpid());
    local_.device = device;
    local_.landing_address = landing;
    local_.landing_bytes = 2 * block_bytes;
    local_.queue_pair = static_cast<uint32_t>(getpid()) ^ (static_cast<uint32_t>(device) << 24);
    local_.packet_sequence = packet_sequence;
    std::snprintf(local_.gid, sizeof(local_.gid), "loopback:%d:%d", host, device);
    std::strncpy(local_.mailbox, mailbox_name.c_str(), sizeof(local_.mailbox) - 1);
    // Device memory crosses processes as an IPC handle of the allocation plus the offset of the landing inside it.
    static_assert(sizeof(cudaIpcMemHandle_t) <= sizeof(local_.landing_handle), "the endpoint holds one IPC handle");
    uint64_t base = 0;
    if (cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(local_.landing_handle), reinterpret_cast<void*>(landing)) ==
            cudaSuccess &&
        allocation_base(landing, &base)) {
        // The handle names the whole allocation; the landing sits at this offset inside it.
        local_.landing_offset = landing - base;
        local_.has_handle = 1;
    } else {
        cudaGetLastError(); // memory that cannot be exported: only same-process peers can connect
        local_.has_handle = 0;
    }
}

loopback_rail::~loopback_rail() {
    try {
        close();
    } catch (...) {
    }
}

void loopback_rail::close() {
    if (closed_) return;
    closed_ = true;
    cudaSetDevice(device_);
    if (stream_) {
        cudaStreamSynchronize(stream_);
        cudaStreamDestroy(stream_);
        stream_ = nullptr;
    }
    if (remote_mapping_ != nullptr) cudaIpcCloseMemHandle(remote_mapping_);
    if (remote_mailbox_ != nullptr && remote_mailbox_ != own_mailbox_) munmap(remote_mailbox_, sizeof(rail_mailbox));
    if (own_mailbox_ != nullptr) {
        munmap(own_mailbox_, sizeof(rail_mailbox));
        shm_unlink(mailbox_name_.c_str());
    }
    remote_mapping_ = nullptr, remote_mailbox_ = nullptr, own_mailbox_ = nullptr;
}

void loopback_rail::connect(rail_endpoint const& remote) {
    check(cudaSetDevice(device_), "cudaSetDevice");
    remote_ = remote;
    if (remote.landing_bytes < 2 * block_bytes_) throw std::runtime_error("rail: the peer's landing buffer is too small");
    if (remote.process == static_cast<uint64_t>(getpid())) {
        remote_landing_ = remote.landing_address;
    } else {
        if (!remote.has_handle) throw std::runtime_error("rail: the peer's landing buffer cannot cross processes");
        cudaIpcMemHandle_t handle;
        std::memcpy(&handle, remote.landing_handle, sizeof(handle));
        check(cudaIpcOpenMemHandle(&remote_mapping_, handle, cudaIpcMemLazyEnablePeerAccess), "opening the peer's landing buffer");
        remote_landing_ = reinterpret_cast<uint64_t>(remote_mapping_) + remote.landing_offset;
    }
    if (std::string(remote.mailbox) == mailbox_name_) {
        remote_mailbox_ = own_mailbox_;
    } else {
        int const descriptor = shm_open(remote.mailbox, O_RDWR, 0600);
        if (descriptor < 0) throw std::runtime_error(std::string("rail: cannot open the peer's mailbox ") + remote.mailbox);
        void* mapping = mmap(nullptr, sizeof(rail_mailbox), PROT_READ | PROT_WRITE, MAP_SHARED, descriptor, 0);
        ::close(descriptor);
        if (mapping == MAP_FAILED) throw std::runtime_error("rail: cannot map the peer's mailbox");
        remote_mailbox_ = static_cast<rail_mailbox*>(mapping);
    }
    connected_ = true;
}

void loopback_rail::post_embeddings(int parity, uint64_t after_stream) {
    if (!connected_) throw std::runtime_error("rail: post before connect");
    if (parity != 0 && parity != 1) throw std::runtime_error("rail: parity is 0 or 1");
    check(cudaSetDevice(device_), "cudaSetDevice");
    // The write may start only after the producer stream has finished the embeddings.
    cudaEvent_t ready;
    check(cudaEventCreateWithFlags(&ready, cudaEventDisableTiming), "creating an event");
    check(cudaEventRecord(ready, reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(after_stream))), "recording an event");
    check(cudaStreamWaitEvent(stream_, ready, 0), "ordering the rail after the producer");
    check(cudaEventDestroy(ready), "destroying an event");
    check(cudaMemcpyAsync(reinterpret_cast<void*>(remote_landing_ + static_cast<uint64_t>(parity) * block_bytes_),
                          reinterpret_cast<void const*>(embeddings_), block_bytes_, cudaMemcpyDefault, stream_),
          "writing the embeddings to the peer");
    uint32_t const status = injected_status_;
    injected_status_ = 0;
    auto* pending = new pending_completion{remote_mailbox_, static_cast<uint32_t>(block_bytes_), status};
    check(cudaLaunchHostFunc(stream_, completion_callback, pending), "queueing the completion");
    ++posted_;
}

void loopback_rail::post_summands(int row, float const* values, int count) {
    if (!connected_) throw std::runtime_error("rail: post before connect");
    if (row < 0 || row >= hosts_) throw std::runtime_error("rail: bad summands row");
    if (count < 1 || count > rail_summand_floats) throw std::runtime_error("rail: a summands row holds 1..16 floats");
    // A reliable connection delivers its writes in the order they were posted. The embeddings' completion is pushed by a
    // host callback on the rail's stream, this one by the calling thread: wait for the stream, so that a completion
    // posted earlier can never arrive after this one (the caller need not have synchronised the device).
    check(cudaSetDevice(device_), "cudaSetDevice");
    check(cudaStreamSynchronize(stream_), "ordering a summands row after the embeddings posted before it");
    for (int i = 0; i < count; ++i) remote_mailbox_->summands[row][i] = values[i];
    std::atomic_thread_fence(std::memory_order_release);
    uint32_t const status = injected_status_;
    injected_status_ = 0;
    push_completion(remote_mailbox_, static_cast<uint32_t>(count * 4), status);
    ++posted_;
}

uint32_t loopback_rail::await_landed(double timeout_seconds) {
    auto const deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(timeout_seconds);
    rail_completion& entry = own_mailbox_->entries[consumed_ % rail_queue_depth];
    while (entry.sequence.load(std::memory_order_acquire) != consumed_ + 1) {
        if (std::chrono::steady_clock::now() > deadline) throw std::runtime_error("rail: timed out waiting for a completion");
        std::this_thread::sleep_for(std::chrono::microseconds(20));
    }
    uint32_t const immediate = entry.immediate, status = entry.status;
    ++consumed_;
    if (status != 0) throw std::runtime_error("rail: completion reported status " + std::to_string(status));
    return immediate;
}

void loopback_rail::read_summands(int row, float* out, int count) const {
    if (row < 0 || row >= hosts_) throw std::runtime_error("rail: bad summands row");
    if (count < 1 || count > rail_summand_floats) throw std::runtime_error("rail: a summands row holds 1..16 floats");
    std::atomic_thread_fence(std::memory_order_acquire);
    for (int i = 0; i < count; ++i) out[i] = own_mailbox_->summands[row][i];
}

void loopback_rail::inject_completion_error(uint32_t status) { injected_status_ = status; }

void loopback_rail::drain() {
    check(cudaSetDevice(device_), "cudaSetDevice");
    check(cudaStreamSynchronize(stream_), "draining the rail");
}

} // namespace sc
