// Public C++ API: one Communicator per process and GPU, three out-of-place collectives.
//
// Parity: reference include/nano_nccl/communicator.h:16-75 — CommunicatorConfig, AllReduceArgs,
// ReduceScatterArgs, AllGatherArgs and the move-only pimpl Communicator with all_reduce /
// reduce_scatter / all_gather / check_async_error / local_rank_count / global_rank_count /
// transport / edge_transport / edge_uses_gdr keep their names, fields and meaning.
// Additions (no counterpart in the reference): algorithm selection, symmetric-memory allocation
// for zero-copy collectives, creation from any Bootstrap, a bounded device wait limit.
#pragma once

#include "nano_nccl/bootstrap.h"
#include "nano_nccl/types.h"

#include <cstddef>
#include <cstdint>
#include <memory>

#include <cuda_runtime.h>

namespace nano_nccl {

struct CommunicatorConfig {
    int device = 0;
    TransportKind transport = TransportKind::Auto;
    // ---- additions ----
    AlgoKind algo = AlgoKind::Auto;          // NANO_NCCL_ALGO overrides when Auto
    std::int64_t wait_timeout_us = 0;        // 0: NANO_NCCL_WAIT_TIMEOUT_US or 20 s
    int enable_multicast = -1;               // -1: NANO_NCCL_NVLS (default on when supported)
    // Framework bindings only: accept the default (null) stream and exact in-place AllReduce
    // (send_buffer == recv_buffer), which the reference API rejects.
    bool relaxed_validation = false;
};

struct AllReduceArgs {
    const void* send_buffer = nullptr;
    void* recv_buffer = nullptr;
    cudaStream_t stream = nullptr;
    std::size_t count = 0;  // elements in and out, per rank
    DType dtype = DType::Float;
    RedOp redop = RedOp::Sum;
};

struct ReduceScatterArgs {
    const void* send_buffer = nullptr;
    void* recv_buffer = nullptr;
    cudaStream_t stream = nullptr;
    std::size_t recv_count = 0;  // output elements per rank; input holds recv_count * ranks
    DType dtype = DType::Float;
    RedOp redop = RedOp::Sum;
};

struct AllGatherArgs {
    const void* send_buffer = nullptr;
    void* recv_buffer = nullptr;
    cudaStream_t stream = nullptr;
    std::size_t send_count = 0;  // input elements per rank; output holds send_count * ranks
    DType dtype = DType::Float;
};

// Counters a caller can read to see which device path ran (observability; tests assert on them).
struct CommunicatorStats {
    std::uint64_t launches = 0;
    std::uint64_t oneshot = 0;
    std::uint64_t twoshot = 0;
    std::uint64_t nvls = 0;
    std::uint64_t ring = 0;
    std::uint64_t zero_copy = 0;  // collectives that ran without staging copies
    std::uint64_t local_only = 0; // single-rank degenerate copies
    std::uint64_t pipelined = 0;  // collectives that took the software-pipelined large-message kernels
};

namespace collective {
class CommunicatorFactory;
}

class Communicator {
public:
    Communicator(const Communicator&) = delete;
    Communicator& operator=(const Communicator&) = delete;
    Communicator(Communicator&&) noexcept;
    Communicator& operator=(Communicator&&) noexcept;
    ~Communicator();

    void all_reduce(const AllReduceArgs& args);
    void reduce_scatter(const ReduceScatterArgs& args);
    void all_gather(const AllGatherArgs& args);
    // Throws the first latched asynchronous failure (device wait limit reached, proxy error).
    void check_async_error() const;
    int local_rank_count() const noexcept;
    int global_rank_count() const noexcept;
    TransportKind transport() const noexcept;
    // Backend of the directed ring edge source_global_rank -> (source_global_rank + 1) % ranks.
    TransportKind edge_transport(int source_global_rank) const;
    // True when a directed RDMA edge uses registered GPU FIFO memory.
    bool edge_uses_gdr(int source_global_rank) const;

    // ---- additions ----
    int rank() const noexcept;
    int device() const noexcept;
    bool multicast_available() const noexcept;
    bool relaxed_validation() const noexcept;
    // Collective call: every rank allocates the same size in the same order.  The returned
    // pointer is ordinary device memory on this rank that peers can address directly, so
    // collectives whose buffers both come from here skip the staging copies.
    void* symmetric_alloc(std::size_t bytes);
    void symmetric_free(void* ptr);
    bool is_symmetric(const void* ptr, std::size_t bytes) const noexcept;
    // Collective.  Makes a buffer the caller allocated with cudaMalloc (or a tensor of a framework's caching
    // allocator) addressable by the peers, so that collectives whose send and receive buffers both lie inside
    // registered or symmetric memory take the zero-copy kernels (peer loads and stores; no multicast).  Every
    // rank passes its own 16-byte aligned pointer and the same size.  The buffer must stay allocated until
    // deregister_buffer (also collective) or the destruction of the communicator.
    void register_buffer(void* ptr, std::size_t bytes);
    void deregister_buffer(void* ptr);
    // Peer view of a symmetric pointer (rank == own rank returns ptr itself).
    void* peer_pointer(const void* ptr, int peer_rank) const;
    // Multicast (NVLS) view of a symmetric pointer; nullptr when multicast is unavailable.
    void* multicast_pointer(const void* ptr) const;
    // Device-side barrier over all ranks on `stream` (bounded wait; errors latch asynchronously).
    void barrier(cudaStream_t stream);
    void set_algo(AlgoKind algo) noexcept;
    // > 0: use exactly this many CTAs for every collective (tuning); 0: back to the tuner table.
    void set_grid_override(int ctas) noexcept;
    AlgoKind last_algo() const noexcept;
    CommunicatorStats stats() const noexcept;
    Bootstrap& bootstrap() const;

    class Impl;  // defined by the library; opaque to callers

private:
    explicit Communicator(std::unique_ptr<Impl> impl);
    std::unique_ptr<Impl> impl_;
    friend class collective::CommunicatorFactory;
    friend class FusedGemmContext;
};

// Creates a communicator over any control plane.  Collective: every rank of `bootstrap` calls it.
// The communicator keeps the bootstrap alive for its own lifetime.
std::unique_ptr<Communicator> create_communicator(std::shared_ptr<Bootstrap> bootstrap,
                                                  const CommunicatorConfig& config);

}  // namespace nano_nccl
