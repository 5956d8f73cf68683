#include "transport/rdma/rdma_proxy.h"

#include "core/error.h"
#include "core/numa.h"
#include "transport/simple/step.h"

#include <arpa/inet.h>
#include <immintrin.h>

#include <cstring>

namespace nano_nccl::rdma {

using simple::host_load_step;
using simple::host_store_step;

// ------------------------------------------------------------------------------------------------
RdmaGdrReceiveFlush::RdmaGdrReceiveFlush(bool fifo_in_device_memory, int ordering) {
    if (!fifo_in_device_memory) return;
    if (ordering < 0) {
        int device = 0, value = 0;
        if (cudaGetDevice(&device) == cudaSuccess &&
            cudaDeviceGetAttribute(&value, cudaDevAttrGPUDirectRDMAWritesOrdering, device) == cudaSuccess) {
            ordering = value;
        } else {
            cudaGetLastError();
            ordering = cudaGPUDirectRDMAWritesOrderingNone;
        }
    }
    // "Owner" (and stronger) ordering makes NIC writes visible to the owning GPU without a flush.
    required_ = ordering < cudaGPUDirectRDMAWritesOrderingOwner;
}

bool RdmaGdrReceiveFlush::flush(std::string* error) {
    if (!required_) return true;
    const int rc = flush_fn_ ? flush_fn_()
                             : static_cast<int>(cudaDeviceFlushGPUDirectRDMAWrites(
                                   cudaFlushGPUDirectRDMAWritesTargetCurrentDevice, cudaFlushGPUDirectRDMAWritesToOwner));
    if (rc != 0) {
        if (error != nullptr) *error = format_message("GPUDirect RDMA write flush failed (code %d)", rc);
        return false;
    }
    ++flushes_;
    return true;
}

// ------------------------------------------------------------------------------------------------
RdmaSendProxy::RdmaSendProxy(ProxyIdentity id, ProxyFifo fifo, QueuePair* qp, MemoryRegion* fifo_mr,
                             AsyncErrorState* errors, RdmaProxyOptions options, volatile RdmaCtsSlot* cts)
    : id_(id), fifo_(fifo), qp_(qp), mr_(fifo_mr), errors_(errors), options_(options), cts_(cts) {
    next_post_ = host_load_step(fifo_.head);
    completed_.store(next_post_, std::memory_order_relaxed);
    timeline_.enable(options.timeline);
    NANO_REQUIRE_ARG(!options.use_write || cts != nullptr, "the WRITE data plane needs a CTS FIFO");
}

void RdmaSendProxy::fail(std::uint64_t step, const std::string& reason) {
    failed_ = true;
    if (errors_ != nullptr) {
        errors_->record(format_message("rdma send proxy failure source=%d destination=%d channel=%d step=%llu: %s",
                                       id_.source, id_.destination, id_.channel,
                                       static_cast<unsigned long long>(step), reason.c_str()));
    }
}

void RdmaSendProxy::retire_through(std::uint64_t step) {
    // RC completes in order: everything up to `step` is done, posted or elided.
    while (!inflight_.empty() && inflight_.front().step <= step) {
        completed_.store(inflight_.front().step + simple::kSliceSteps, std::memory_order_release);
        inflight_.pop_front();
        inflight_count_.store(inflight_.size(), std::memory_order_release);
    }
}

// Callable from any thread (teardown asks while the progress thread still runs): reads the published counters only.
bool RdmaSendProxy::drained() const {
    return failed_.load(std::memory_order_acquire) ||
           (inflight_count_.load(std::memory_order_acquire) == 0 &&
            host_load_step(fifo_.tail) <= completed_.load(std::memory_order_acquire));
}

bool RdmaSendProxy::progress() {
    if (failed_ || (errors_ != nullptr && errors_->has_error())) return false;
    bool moved = false;
    try {
        // ---- post while the window has room and the kernel has produced slices
        while (static_cast<int>(inflight_.size()) < kMaxInflight) {
            const std::uint64_t tail = host_load_step(fifo_.tail);
            if (tail < next_post_ + simple::kSliceSteps) break;
            const std::size_t slot = next_post_ % simple::kFifoSteps;
            const std::uint32_t bytes = fifo_.slot_bytes[slot];
            NANO_REQUIRE(bytes <= simple::kSliceBytes, "slot announces %u bytes, above the slice capacity", bytes);
            if (bytes == 0) {
                // zero-byte branch: nothing goes to the NIC
                inflight_.push_back({next_post_, false});
                inflight_count_.store(inflight_.size(), std::memory_order_release);
                ++zero_payload_posts_;
            } else {
                const bool more = tail >= next_post_ + 2 * simple::kSliceSteps &&
                                  static_cast<int>(inflight_.size()) + 1 < kMaxInflight;
                const bool next_is_zero = more && fifo_.slot_bytes[(next_post_ + simple::kSliceSteps) % simple::kFifoSteps] == 0;
                const bool signaled = !more || next_is_zero || (posts_ % kSignalEvery) == kSignalEvery - 1;
                Sge sge{fifo_.fifo + slot * simple::kStepBytes, bytes, mr_->lkey()};  // straight from the FIFO
                if (options_.use_write) {
                    volatile RdmaCtsSlot& grant = cts_[(next_post_ / simple::kSliceSteps) % kCtsSlots];
                    if (!(grant.ready != 0 && grant.step_tag == next_post_)) break;  // no clear-to-send yet
                    __atomic_thread_fence(__ATOMIC_ACQUIRE);
                    NANO_REQUIRE(bytes <= grant.nbytes, "slice of %u bytes exceeds the granted %u bytes", bytes, grant.nbytes);
                    qp_->post_write_imm(next_post_, sge, grant.raddr, grant.rkey, htonl(bytes), signaled);
                    grant.ready = 0;  // right after the post: the grant is spent
                } else {
                    qp_->post_send(next_post_, sge, signaled, false);
                }
                inflight_.push_back({next_post_, true});
                inflight_count_.store(inflight_.size(), std::memory_order_release);
                ++posts_;
                if (signaled) ++signaled_posts_;
                timeline_.depth(TimelineDepth::Inflight, static_cast<unsigned>(inflight_.size()));
            }
            next_post_ += simple::kSliceSteps;
            moved = true;
        }
        // ---- zero-byte slices at the head of the completion order retire on the host
        while (!inflight_.empty() && !inflight_.front().posted) {
            completed_.store(inflight_.front().step + simple::kSliceSteps, std::memory_order_release);
            inflight_.pop_front();
            inflight_count_.store(inflight_.size(), std::memory_order_release);
            moved = true;
        }
        // ---- harvest completions
        WorkCompletion wc[kPollBatch];
        const int n = qp_->poll(wc, kPollBatch);
        for (int i = 0; i < n; ++i) {
            if (!wc[i].ok) {
                fail(wc[i].wr_id, "work completion failed: " + wc[i].error);
                return true;
            }
            if (wc[i].opcode == WcOpcode::Send || wc[i].opcode == WcOpcode::Write) {
                retire_through(wc[i].wr_id);
                moved = true;
            }
        }
        while (!inflight_.empty() && !inflight_.front().posted) {
            completed_.store(inflight_.front().step + simple::kSliceSteps, std::memory_order_release);
            inflight_.pop_front();
            inflight_count_.store(inflight_.size(), std::memory_order_release);
        }
        const std::uint64_t done = completed_.load(std::memory_order_relaxed);
        if (host_load_step(fifo_.head) != done) host_store_step(fifo_.head, done);
    } catch (const std::exception& e) {
        fail(next_post_, e.what());
        return true;
    }
    return moved;
}

// ------------------------------------------------------------------------------------------------
RdmaRecvProxy::RdmaRecvProxy(ProxyIdentity id, ProxyFifo fifo, QueuePair* qp, MemoryRegion* fifo_mr,
                             AsyncErrorState* errors, RdmaProxyOptions options, RdmaGdrReceiveFlush flush,
                             RdmaCtsSlot* cts_staging, MemoryRegion* cts_staging_mr, std::uint64_t remote_cts_addr,
                             std::uint32_t remote_cts_rkey, void* scratch, MemoryRegion* scratch_mr)
    : id_(id), fifo_(fifo), qp_(qp), mr_(fifo_mr), errors_(errors), options_(options), flush_(std::move(flush)),
      cts_staging_(cts_staging), cts_staging_mr_(cts_staging_mr), remote_cts_addr_(remote_cts_addr),
      remote_cts_rkey_(remote_cts_rkey), scratch_(scratch), scratch_mr_(scratch_mr) {
    next_post_ = next_done_ = host_load_step(fifo_.tail);
    NANO_REQUIRE_ARG(!options.use_write || (cts_staging != nullptr && cts_staging_mr != nullptr && scratch != nullptr &&
                                            scratch_mr != nullptr),
                     "the WRITE data plane needs CTS staging records and a scratch receive buffer");
}

void RdmaRecvProxy::fail(std::uint64_t step, const std::string& reason) {
    failed_ = true;
    if (errors_ != nullptr) {
        errors_->record(format_message("rdma recv proxy failure source=%d destination=%d channel=%d step=%llu: %s",
                                       id_.source, id_.destination, id_.channel,
                                       static_cast<unsigned long long>(step), reason.c_str()));
    }
}

bool RdmaRecvProxy::progress() {
    if (failed_ || (errors_ != nullptr && errors_->has_error())) return false;
    bool moved = false;
    try {
        // ---- grant / pre-post every slot pair the consumer has freed (credit back-pressure)
        while (next_post_ + simple::kSliceSteps <= host_load_step(fifo_.head) + simple::kFifoSteps) {
            const std::size_t slot = next_post_ % simple::kFifoSteps;
            char* slot_addr = fifo_.fifo + slot * simple::kStepBytes;
            if (options_.use_write) {
                // scratch receive harvests the immediate; the payload lands by RDMA write
                qp_->post_recv(next_post_, Sge{scratch_, 1, scratch_mr_->lkey()});
                RdmaCtsSlot& rec = cts_staging_[(next_post_ / simple::kSliceSteps) % kCtsSlots];
                rec.raddr = reinterpret_cast<std::uint64_t>(slot_addr);
                rec.rkey = mr_->rkey();
                rec.nbytes = static_cast<std::uint32_t>(simple::kSliceBytes);
                rec.step_tag = next_post_;
                rec.ready = 1;
                const bool inline_ok = sizeof(RdmaCtsSlot) <= qp_->max_inline();
                const std::uint64_t raddr = remote_cts_addr_ +
                                            ((next_post_ / simple::kSliceSteps) % kCtsSlots) * sizeof(RdmaCtsSlot);
                qp_->post_write(next_post_, Sge{&rec, sizeof(RdmaCtsSlot), cts_staging_mr_->lkey()}, raddr,
                                remote_cts_rkey_, /*signaled=*/false, inline_ok);
                ++cts_posts_;
                if (inline_ok) ++cts_inline_posts_;
            } else {
                qp_->post_recv(next_post_, Sge{slot_addr, static_cast<std::uint32_t>(simple::kSliceBytes), mr_->lkey()});
            }
            next_post_ += simple::kSliceSteps;
            moved = true;
        }
        // ---- completions: flush (if the device needs it) -> slot size -> tail
        WorkCompletion wc[kPollBatch];
        const int n = qp_->poll(wc, kPollBatch);
        for (int i = 0; i < n; ++i) {
            if (!wc[i].ok) {
                fail(wc[i].wr_id, "work completion failed: " + wc[i].error);
                return true;
            }
            if (wc[i].opcode != WcOpcode::Recv && wc[i].opcode != WcOpcode::RecvImm) continue;  // CTS write completions
            NANO_REQUIRE(wc[i].wr_id == next_done_, "receive completed out of order (step %llu, expected %llu)",
                         static_cast<unsigned long long>(wc[i].wr_id), static_cast<unsigned long long>(next_done_));
            const std::uint32_t bytes = wc[i].opcode == WcOpcode::RecvImm ? ntohl(wc[i].imm_be) : wc[i].byte_len;
            NANO_REQUIRE(bytes <= simple::kSliceBytes, "received %u bytes, above the slice capacity", bytes);
            std::string flush_error;
            if (!flush_.flush(&flush_error)) {
                fail(next_done_, flush_error);
                return true;
            }
            fifo_.slot_bytes[next_done_ % simple::kFifoSteps] = bytes;
            next_done_ += simple::kSliceSteps;
            ++received_;
            host_store_step(fifo_.tail, next_done_);
            moved = true;
        }
    } catch (const std::exception& e) {
        fail(next_done_, e.what());
        return true;
    }
    return moved;
}

// ------------------------------------------------------------------------------------------------
RdmaProgressEngine::RdmaProgressEngine(bool shared, int numa_node, AsyncErrorState* errors)
    : shared_(shared), numa_node_(numa_node), errors_(errors) {}

RdmaProgressEngine::~RdmaProgressEngine() { stop(); }

void RdmaProgressEngine::loop(std::vector<RdmaProxy*> recv, std::vector<RdmaProxy*> send) {
    try {
        pin_current_thread_to_numa_node(numa_node_);
    } catch (const std::exception& e) {
        if (errors_ != nullptr) errors_->record(std::string("rdma progress thread: ") + e.what());
        return;
    }
    while (!stop_.load(std::memory_order_acquire)) {
        bool moved = false;
        for (RdmaProxy* p : recv) moved = p->progress() || moved;  // receives first: frees the peer sooner
        for (RdmaProxy* p : send) moved = p->progress() || moved;
        if (!moved) _mm_pause();
    }
}

void RdmaProgressEngine::start() {
    if (!threads_.empty()) return;
    if (shared_) {
        threads_.emplace_back([this] { loop(recv_, send_); });
    } else {
        for (RdmaProxy* p : recv_) threads_.emplace_back([this, p] { loop({p}, {}); });
        for (RdmaProxy* p : send_) threads_.emplace_back([this, p] { loop({}, {p}); });
    }
}

void RdmaProgressEngine::stop() {
    stop_.store(true, std::memory_order_release);
    for (auto& t : threads_) if (t.joinable()) t.join();
    threads_.clear();
}

}  // namespace nano_nccl::rdma
