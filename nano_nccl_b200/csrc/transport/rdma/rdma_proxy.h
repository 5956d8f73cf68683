// Host-side engines of the RDMA transport: per (edge, channel) send and receive proxies that
// move Simple-protocol slices between a registered FIFO and a reliable-connected queue pair, the
// GPUDirect receive flush, and the progress engine that drives them.
//
// Parity: reference src/transport/rdma/rdma_proxy.{h,cc}, rdma_gdr.{h,cc}, rdma_progress.{h,cc}.
// Kept:
//  * two data planes: SEND/RECV (receives pre-posted for whole slot pairs, the completion's byte
//    count is the slice size) and WRITE_WITH_IMM + CTS (the receiver grants each free slot pair by
//    writing a 32-byte clear-to-send record into the sender's CTS FIFO, inline when it fits; the
//    sender waits for `ready && step_tag == step`, posts RDMA_WRITE_WITH_IMM with the byte count
//    as big-endian immediate and clears `ready` right after posting; the receiver harvests the
//    immediate through a 1-byte scratch receive);
//  * up to 4 slices in flight per edge, selective signalling (every 4th post, when the window
//    fills, at the end of a burst, before a zero-byte slice) with wr_id = absolute step so that
//    one completion retires every earlier send (RC keeps order);
//  * zero-byte slices are never posted: they are retired on the host when they reach the head of
//    the completion order;
//  * the SGE points into the registered FIFO itself (no bounce copy);
//  * receive order: completion -> GPUDirect flush (when the device needs it) -> slot size ->
//    `recv_tail` release-store;
//  * first-error latch: message, device-visible abort word, flag.
#pragma once

#include "transport/rdma/rdma_timeline.h"
#include "transport/rdma/verbs.h"
#include "transport/simple/protocol.h"
#include "transport/socket/socket_proxy.h"

#include <atomic>
#include <deque>
#include <functional>
#include <thread>
#include <vector>

namespace nano_nccl::rdma {

using AsyncErrorState = socket_transport::SocketAsyncErrorState;
using socket_transport::ProxyFifo;
using socket_transport::ProxyIdentity;

constexpr int kMaxInflight = simple::kFifoSteps / simple::kSliceSteps;  // 4
constexpr int kCtsSlots = kMaxInflight;
constexpr int kSignalEvery = 4;
constexpr int kPollBatch = 16;

// Decides whether data written by the NIC into GPU memory must be flushed before the GPU may be
// told about it, and does it.  `ordering` is cudaDevAttrGPUDirectRDMAWritesOrdering (-1: query the
// current device); a flush is needed for device memory when ordering is below "owner".
class RdmaGdrReceiveFlush {
public:
    RdmaGdrReceiveFlush(bool fifo_in_device_memory, int ordering = -1);
    bool required() const noexcept { return required_; }
    // No-op when not required.  Returns false (with *error set) if the flush call failed.
    bool flush(std::string* error);
    std::uint64_t flushes() const noexcept { return flushes_; }
    // Test seam: replaces the CUDA call.
    void set_flush_function(std::function<int()> fn) { flush_fn_ = std::move(fn); }

private:
    bool required_ = false;
    std::uint64_t flushes_ = 0;
    std::function<int()> flush_fn_;
};

struct RdmaProxyOptions {
    bool use_write = false;     // WRITE_WITH_IMM + CTS data plane
    bool timeline = false;
};

class RdmaProxy {
public:
    virtual ~RdmaProxy() = default;
    // One non-blocking pass.  Returns true if anything moved.
    virtual bool progress() = 0;
    virtual bool failed() const = 0;
};

class RdmaSendProxy final : public RdmaProxy {
public:
    // `fifo_mr` covers fifo.fifo.  WRITE mode: `cts` are this side's kCtsSlots CTS records (the
    // peer writes them), `remote_fifo_*` describe the peer's receive FIFO.
    RdmaSendProxy(ProxyIdentity id, ProxyFifo fifo, QueuePair* qp, MemoryRegion* fifo_mr, AsyncErrorState* errors,
                  RdmaProxyOptions options, volatile RdmaCtsSlot* cts = nullptr);
    bool progress() override;
    bool failed() const override { return failed_; }
    bool drained() const;
    std::uint64_t posts() const noexcept { return posts_; }
    std::uint64_t zero_payload_posts() const noexcept { return zero_payload_posts_; }
    std::uint64_t signaled_posts() const noexcept { return signaled_posts_; }
    const RdmaProxyTimeline& timeline() const noexcept { return timeline_; }

private:
    struct Flight {
        std::uint64_t step;
        bool posted;   // false: zero-byte slice, retired on the host
    };
    void fail(std::uint64_t step, const std::string& reason);
    void retire_through(std::uint64_t step);

    ProxyIdentity id_;
    ProxyFifo fifo_;
    QueuePair* qp_;
    MemoryRegion* mr_;
    AsyncErrorState* errors_;
    RdmaProxyOptions options_;
    volatile RdmaCtsSlot* cts_;
    std::deque<Flight> inflight_;                  // touched by the progress thread only
    std::atomic<std::size_t> inflight_count_{0};   // its size, for drained() on another thread
    std::uint64_t next_post_ = 0;
    std::atomic<std::uint64_t> completed_{0};      // written by the progress thread, read by drained()
    std::uint64_t posts_ = 0, zero_payload_posts_ = 0, signaled_posts_ = 0;
    std::atomic<bool> failed_{false};
    RdmaProxyTimeline timeline_;
};

class RdmaRecvProxy final : public RdmaProxy {
public:
    // WRITE mode: `cts_staging` are kCtsSlots local records inside `cts_staging_mr` used as the
    // source of the CTS writes; `remote_cts_*` is the sender's CTS FIFO.
    RdmaRecvProxy(ProxyIdentity id, ProxyFifo fifo, QueuePair* qp, MemoryRegion* fifo_mr, AsyncErrorState* errors,
                  RdmaProxyOptions options, RdmaGdrReceiveFlush flush, RdmaCtsSlot* cts_staging = nullptr,
                  MemoryRegion* cts_staging_mr = nullptr, std::uint64_t remote_cts_addr = 0,
                  std::uint32_t remote_cts_rkey = 0, void* scratch = nullptr, MemoryRegion* scratch_mr = nullptr);
    bool progress() override;
    bool failed() const override { return failed_; }
    std::uint64_t received() const noexcept { return received_; }
    std::uint64_t cts_posts() const noexcept { return cts_posts_; }
    std::uint64_t cts_inline_posts() const noexcept { return cts_inline_posts_; }
    const RdmaGdrReceiveFlush& flush_state() const noexcept { return flush_; }

private:
    void fail(std::uint64_t step, const std::string& reason);

    ProxyIdentity id_;
    ProxyFifo fifo_;
    QueuePair* qp_;
    MemoryRegion* mr_;
    AsyncErrorState* errors_;
    RdmaProxyOptions options_;
    RdmaGdrReceiveFlush flush_;
    RdmaCtsSlot* cts_staging_;
    MemoryRegion* cts_staging_mr_;
    std::uint64_t remote_cts_addr_;
    std::uint32_t remote_cts_rkey_;
    void* scratch_;
    MemoryRegion* scratch_mr_;
    std::uint64_t next_post_ = 0;   // next step to grant / pre-post
    std::uint64_t next_done_ = 0;   // next step expected to complete
    std::uint64_t received_ = 0, cts_posts_ = 0, cts_inline_posts_ = 0;
    std::atomic<bool> failed_{false};
};

// Drives proxies: one shared thread (receives first, then sends, pause when idle) or one thread
// per proxy.  NUMA-pinned; a pinning failure is latched as an asynchronous error.
class RdmaProgressEngine {
public:
    RdmaProgressEngine(bool shared, int numa_node, AsyncErrorState* errors);
    ~RdmaProgressEngine();
    void add_recv(RdmaProxy* proxy) { recv_.push_back(proxy); }
    void add_send(RdmaProxy* proxy) { send_.push_back(proxy); }
    void start();
    void stop();
    int thread_count() const noexcept { return static_cast<int>(threads_.size()); }

private:
    void loop(std::vector<RdmaProxy*> recv, std::vector<RdmaProxy*> send);
    bool shared_;
    int numa_node_;
    AsyncErrorState* errors_;
    std::vector<RdmaProxy*> recv_, send_;
    std::vector<std::thread> threads_;
    std::atomic<bool> stop_{false};
};

}  // namespace nano_nccl::rdma
