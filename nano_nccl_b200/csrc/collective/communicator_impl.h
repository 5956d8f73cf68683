// Private state of a Communicator.  See communicator.cc for the behaviour.
#pragma once

#include "bootstrap/fd_channel.h"
#include "collective/tuner.h"
#include "core/buffer.h"
#include "core/numa.h"
#include "core/stream.h"
#include "kernels/launch.h"
#include "nano_nccl/communicator.h"
#include "symm/symmetric_memory.h"
#include "topology/topology.h"

#include <memory>
#include <string>
#include <vector>

namespace nano_nccl {

// The Ring/Simple fallback data plane (multi-channel FIFO ring over P2P / SHM / socket / RDMA
// edges).  Implemented in transport/ring_path.*; the communicator only sees this interface.
class RingPath {
public:
    virtual ~RingPath() = default;
    virtual void run(CollectiveKind kind, const void* send, void* recv, std::size_t count,
                     DType dtype, RedOp op, cudaStream_t stream) = 0;
    virtual bool async_error(std::string* message) const = 0;
    virtual bool edge_uses_gdr(int source_rank) const = 0;
};

class Communicator::Impl {
public:
    Impl(std::shared_ptr<Bootstrap> bootstrap, const CommunicatorConfig& config);
    ~Impl();

    void all_reduce(const AllReduceArgs& args);
    void reduce_scatter(const ReduceScatterArgs& args);
    void all_gather(const AllGatherArgs& args);
    void barrier(cudaStream_t stream);
    void check_async_error() const;
    void* symmetric_alloc(std::size_t bytes);
    void symmetric_free(void* ptr);
    void register_buffer(void* ptr, std::size_t bytes);
    void* peer_pointer(const void* ptr, int peer) const;
    void* multicast_pointer(const void* ptr) const;
    SymmetricMemory* find_symmetric(const void* ptr, std::size_t bytes) const noexcept;
    TransportKind edge_transport(int source) const;
    bool edge_uses_gdr(int source) const;
    bool multicast_available() const noexcept { return arena_ != nullptr && arena_->multicast() != nullptr; }
    bool config_relaxed() const noexcept { return config_.relaxed_validation; }
    // Pushes go through the switch's multicast only when it saves stores (more than one peer).
    bool push_multicast() const noexcept { return multicast_available() && nranks_ > 2; }
    // Serialises this launch after the previous collective when the stream changed.
    void order_after_previous(cudaStream_t stream);
    const dev::CommDev& device_context() const noexcept { return dev_; }
    void set_ring(std::unique_ptr<RingPath> ring) { ring_ = std::move(ring); }

    std::shared_ptr<Bootstrap> bootstrap_;
    CommunicatorConfig config_;
    int rank_ = 0;
    int nranks_ = 1;
    int device_ = 0;
    std::int64_t timeout_us_ = 0;
    bool relaxed_validation_ = false;
    bool nvlink_path_ = false;
    int debug_level_ = 0;        // NANO_NCCL_DEBUG: unset / 0 = quiet, info = one line at creation, trace = one line per collective
    std::size_t tile_cap_ = 0;  // NANO_NCCL_TILE_BYTES: cap on the tile size (0: as large as staging allows)
    std::size_t pipe_min_bytes_ = 0;   // NANO_NCCL_PIPE_MIN_BYTES: smallest message of the software-pipelined kernels (0: off)
    std::size_t pipe_tile_bytes_ = 0;  // NANO_NCCL_PIPE_TILE_BYTES: their tile size (0: a sixteenth of a CTA's region)
    int pipe_depth_ = 0;               // NANO_NCCL_PIPE_DEPTH: iterations between a tile's stages (0: the built-in choice)
    AlgoKind pipe_algo_ = AlgoKind::Auto;  // NANO_NCCL_PIPE_ALGO: auto / twoshot / nvls for the pipelined AllReduce
    bool push_tma_ = false;  // NANO_NCCL_PUSH_TMA=1: AllGather pushes through TMA bulk copies (experimental)
    bool debug_signatures_ = false;  // NANO_NCCL_DEBUG_SIGNATURES=1: ranks compare descriptors before every call
    std::uint64_t call_sequence_ = 0;
    bool skew_ = false;  // NANO_NCCL_SKEW=1: half-tile phase shift of odd CTAs in two-phase kernels
    std::vector<RankInfo> ranks_;
    ProcessTopology topology_;
    RingTransportPlan plan_;
    std::unique_ptr<FdChannel> fds_;
    std::unique_ptr<SymmetricMemory> arena_;
    RawDeviceBuffer state_;
    RawDeviceBuffer barrier_words_;  // send + receive word of barrier() on the ring transports, made on first use
    MappedU32Array status_;
    MappedU32Array abort_;
    dev::CommDev dev_{};
    std::unique_ptr<SymmetricMemory> ll_arena_;  // staging of the flag-in-data kernels, when enabled
    dev::LLDev ll_dev_{};
    std::size_t ll_max_bytes_ = 0;               // NANO_NCCL_LL_MAX_BYTES: largest message that takes them (0: off)
    std::unique_ptr<Tuner> tuner_;
    std::vector<std::unique_ptr<SymmetricMemory>> heap_;
    std::unique_ptr<RingPath> ring_;
    Event completion_;
    cudaStream_t last_stream_ = nullptr;
    bool has_last_stream_ = false;
    AlgoKind last_algo_ = AlgoKind::Auto;
    CommunicatorStats stats_{};
    mutable std::string async_error_;

private:
    void fill_device_context();
    void validate_args(const void* send, void* recv, cudaStream_t stream, std::size_t count,
                       std::size_t send_elems, std::size_t recv_elems, DType dtype, int redop,
                       bool allow_exact_in_place) const;
    void local_copy(const void* send, void* recv, std::size_t bytes, cudaStream_t stream);
    void check_signature(CollectiveKind kind, std::size_t count, DType dtype, int redop, bool in_place);
    void run_ring(CollectiveKind kind, const void* send, void* recv, std::size_t count, DType dtype,
                  RedOp op, cudaStream_t stream);
};

namespace collective {
class CommunicatorFactory {
public:
    static std::unique_ptr<Communicator> create(std::shared_ptr<Bootstrap> bootstrap,
                                                const CommunicatorConfig& config);
    static Communicator::Impl& impl(Communicator& communicator);
};
}  // namespace collective

}  // namespace nano_nccl
