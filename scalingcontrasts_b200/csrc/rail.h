// The rail's types: the endpoint record that two sides exchange, the receiver's mailbox (completion queue and
// summands table), and the loopback rail itself. See rail.cpp.
#pragma once

#include <atomic>
#include <cstdint>
#include <string>

#include <cuda_runtime.h>

namespace sc {

constexpr int rail_queue_depth = 64;
constexpr int rail_max_hosts = 64;
constexpr int rail_summand_floats = 16; // one row of loss summands

// What one side publishes so that the other can write to it. Plain bytes: it crosses processes through a file.
struct rail_endpoint {
    char gid[32];
    uint64_t process;
    int32_t device;
    uint32_t has_handle;
    uint64_t landing_address;
    uint64_t landing_offset;
    uint64_t landing_bytes;
    unsigned char landing_handle[64];
    char mailbox[64];
    uint32_t queue_pair;
    uint32_t packet_sequence;
};

struct rail_completion {
    std::atomic<uint64_t> sequence;
    uint32_t immediate;
    uint32_t status;
};

struct rail_mailbox {
    std::atomic<uint64_t> head;
    rail_completion entries[rail_queue_depth];
    float summands[rail_max_hosts][rail_summand_floats];
};

class loopback_rail {
  public:
    loopback_rail(int device, uint64_t embeddings, uint64_t block_bytes, uint64_t landing, int hosts, int host,
                  std::string const& mailbox_name, uint32_t packet_sequence);
    ~loopback_rail();
    loopback_rail(loopback_rail const&) = delete;
    loopback_rail& operator=(loopback_rail const&) = delete;

    rail_endpoint const& local() const { return local_; }
    void connect(rail_endpoint const& remote);
    // Writes this side's embeddings into the peer's landing[parity] once `after_stream` has produced them.
    void post_embeddings(int parity, uint64_t after_stream);
    // Writes `count` floats (at most rail_summand_floats) into row `row` of the peer's summands table.
    void post_summands(int row, float const* values, int count);
    // Consumes one completion; returns its immediate data. Throws on a timeout or on an error completion.
    uint32_t await_landed(double timeout_seconds);
    void read_summands(int row, float* out, int count) const;
    // The next completion this side produces carries `status` instead of success (host-side fault injection).
    void inject_completion_error(uint32_t status);
    void drain();
    void close();
    uint64_t posted() const { return posted_; }
    uint64_t consumed() const { return consumed_; }

  private:
    int device_;
    uint64_t embeddings_, block_bytes_, landing_;
    int hosts_, host_;
    std::string mailbox_name_;
    rail_endpoint local_{}, remote_{};
    rail_mailbox* own_mailbox_ = nullptr;
    rail_mailbox* remote_mailbox_ = nullptr;
    void* remote_mapping_ = nullptr;
    uint64_t remote_landing_ = 0;
    cudaStream_t stream_ = nullptr;
    bool connected_ = false, closed_ = false;
    uint32_t injected_status_ = 0;
    uint64_t posted_ = 0, consumed_ = 0;
};

} // namespace sc
