// In-process loopback provider of the verbs interface (unit tests of the RDMA proxies).
// Reliable-connected semantics: a send consumes the oldest posted receive of the peer; data and
// completions are delivered in posting order; an RDMA write checks the remote key and bounds; a
// write with immediate also consumes a receive and reports the immediate; unsignaled sends
// produce no completion.  A send with no receive posted waits (receiver-not-ready) and is retried
// at the next poll of either side, as an RC QP with an infinite RNR retry count would.
#include "transport/rdma/verbs.h"

#include "core/error.h"

#include <atomic>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>

namespace nano_nccl::rdma {

namespace {

struct Fabric {
    std::mutex mutex;
    struct Region { char* base; std::size_t bytes; };
    std::map<std::uint32_t, Region> regions;  // by rkey
    std::atomic<std::uint32_t> next_key{0x1000};
    std::atomic<std::uint32_t> next_qpn{1};
};

class LoopbackMr final : public MemoryRegion {
public:
    LoopbackMr(std::shared_ptr<Fabric> f, void* addr, std::size_t bytes, bool device)
        : fabric_(std::move(f)), addr_(addr), bytes_(bytes), device_(device) {
        key_ = fabric_->next_key.fetch_add(1);
        std::lock_guard<std::mutex> lock(fabric_->mutex);
        fabric_->regions[key_] = {static_cast<char*>(addr), bytes};
    }
    ~LoopbackMr() override {
        std::lock_guard<std::mutex> lock(fabric_->mutex);
        fabric_->regions.erase(key_);
    }
    std::uint32_t lkey() const override { return key_; }
    std::uint32_t rkey() const override { return key_; }
    void* addr() const override { return addr_; }
    std::size_t length() const override { return bytes_; }
    bool is_device_memory() const override { return device_; }
    bool uses_dmabuf() const override { return false; }

private:
    std::shared_ptr<Fabric> fabric_;
    void* addr_;
    std::size_t bytes_;
    bool device_;
    std::uint32_t key_ = 0;
};

class LoopbackQp;
std::mutex g_qp_registry_mutex;
// Never destroyed: a progress thread may still look a peer up while the process runs its exit handlers.
std::map<std::uint32_t, LoopbackQp*>& qp_registry() {
    static auto* registry = new std::map<std::uint32_t, LoopbackQp*>();
    return *registry;
}

class LoopbackQp final : public QueuePair {
public:
    LoopbackQp(std::shared_ptr<Fabric> f, int send_depth, int recv_depth)
        : fabric_(std::move(f)), send_depth_(send_depth), recv_depth_(recv_depth) {
        qpn_ = fabric_->next_qpn.fetch_add(1);
        std::lock_guard<std::mutex> lock(g_qp_registry_mutex);
        qp_registry()[qpn_] = this;
    }
    ~LoopbackQp() override {
        std::lock_guard<std::mutex> lock(g_qp_registry_mutex);
        qp_registry().erase(qpn_);
    }

    void post_send(std::uint64_t wr_id, const Sge& sge, bool signaled, bool) override {
        enqueue({Kind::Send, wr_id, sge, 0, 0, 0, signaled});
    }
    void post_write(std::uint64_t wr_id, const Sge& sge, std::uint64_t raddr, std::uint32_t rkey, bool signaled,
                    bool) override {
        enqueue({Kind::Write, wr_id, sge, raddr, rkey, 0, signaled});
    }
    void post_write_imm(std::uint64_t wr_id, const Sge& sge, std::uint64_t raddr, std::uint32_t rkey,
                        std::uint32_t imm_be, bool signaled) override {
        enqueue({Kind::WriteImm, wr_id, sge, raddr, rkey, imm_be, signaled});
    }
    void post_recv(std::uint64_t wr_id, const Sge& sge) override {
        std::lock_guard<std::mutex> lock(fabric_->mutex);
        NANO_REQUIRE(static_cast<int>(recvs_.size()) < recv_depth_, "loopback qp: receive queue overflow");
        recvs_.push_back({wr_id, sge});
    }
    int poll(WorkCompletion* out, int max) override {
        LoopbackQp* peer = peer_qp();
        std::lock_guard<std::mutex> lock(fabric_->mutex);
        progress_locked(peer);
        if (peer != nullptr) peer->progress_locked(this);
        int n = 0;
        while (n < max && !cq_.empty()) {
            out[n++] = cq_.front();
            cq_.pop_front();
        }
        return n;
    }
    std::uint32_t max_inline() const override { return 64; }
    void fill_local_info(RdmaPeerInfo* info) const override {
        info->qp_num = qpn_;
        info->psn = 0;
        info->lid = 1;
        info->path_mtu = 5;
    }
    void connect(const RdmaPeerInfo& peer) override { peer_qpn_ = peer.qp_num; }

private:
    enum class Kind { Send, Write, WriteImm };
    struct SendWr {
        Kind kind;
        std::uint64_t wr_id;
        Sge sge;
        std::uint64_t raddr;
        std::uint32_t rkey;
        std::uint32_t imm_be;
        bool signaled;
    };
    struct RecvWr {
        std::uint64_t wr_id;
        Sge sge;
    };

    void enqueue(SendWr wr) {
        std::lock_guard<std::mutex> lock(fabric_->mutex);
        NANO_REQUIRE(static_cast<int>(sends_.size()) < send_depth_, "loopback qp: send queue overflow");
        sends_.push_back(wr);
    }

    LoopbackQp* peer_qp() const {
        std::lock_guard<std::mutex> lock(g_qp_registry_mutex);
        auto it = qp_registry().find(peer_qpn_);
        return it == qp_registry().end() ? nullptr : it->second;
    }

    // Executes queued sends in order against `peer` (caller holds the fabric mutex).
    void progress_locked(LoopbackQp* peer) {
        if (peer == nullptr) return;
        while (!sends_.empty()) {
            SendWr& wr = sends_.front();
            WorkCompletion mine;
            mine.wr_id = wr.wr_id;
            mine.opcode = wr.kind == Kind::Send ? WcOpcode::Send : WcOpcode::Write;
            if (wr.kind == Kind::Send || wr.kind == Kind::WriteImm) {
                if (peer->recvs_.empty()) return;  // receiver not ready: retry later, order kept
            }
            if (wr.kind == Kind::Write || wr.kind == Kind::WriteImm) {
                auto it = fabric_->regions.find(wr.rkey);
                const char* dst = reinterpret_cast<const char*>(wr.raddr);
                if (it == fabric_->regions.end() || dst < it->second.base ||
                    dst + wr.sge.length > it->second.base + it->second.bytes) {
                    mine.ok = false;
                    mine.error = "remote access error";
                    cq_.push_back(mine);
                    sends_.pop_front();
                    continue;
                }
                if (wr.sge.length != 0) std::memcpy(const_cast<char*>(dst), wr.sge.addr, wr.sge.length);
            }
            if (wr.kind == Kind::Send) {
                RecvWr rr = peer->recvs_.front();
                peer->recvs_.pop_front();
                WorkCompletion theirs;
                theirs.wr_id = rr.wr_id;
                theirs.opcode = WcOpcode::Recv;
                if (wr.sge.length > rr.sge.length) {
                    theirs.ok = false;
                    theirs.error = "local length error";
                    mine.ok = false;
                    mine.error = "remote invalid request";
                } else {
                    if (wr.sge.length != 0) std::memcpy(rr.sge.addr, wr.sge.addr, wr.sge.length);
                    theirs.byte_len = wr.sge.length;
                }
                peer->cq_.push_back(theirs);
            } else if (wr.kind == Kind::WriteImm) {
                RecvWr rr = peer->recvs_.front();
                peer->recvs_.pop_front();
                WorkCompletion theirs;
                theirs.wr_id = rr.wr_id;
                theirs.opcode = WcOpcode::RecvImm;
                theirs.byte_len = wr.sge.length;
                theirs.imm_be = wr.imm_be;
                peer->cq_.push_back(theirs);
            }
            if (wr.signaled || !mine.ok) cq_.push_back(mine);
            sends_.pop_front();
        }
    }

    std::shared_ptr<Fabric> fabric_;
    int send_depth_, recv_depth_;
    std::uint32_t qpn_ = 0;
    std::uint32_t peer_qpn_ = 0;
    std::deque<SendWr> sends_;
    std::deque<RecvWr> recvs_;
    std::deque<WorkCompletion> cq_;
};

class LoopbackDevice final : public VerbsDevice {
public:
    explicit LoopbackDevice(std::string name) : name_(std::move(name)), fabric_(std::make_shared<Fabric>()) {}
    std::string name() const override { return name_; }
    std::unique_ptr<MemoryRegion> register_host(void* addr, std::size_t bytes) override {
        return std::make_unique<LoopbackMr>(fabric_, addr, bytes, false);
    }
    std::unique_ptr<MemoryRegion> register_device(void* addr, std::size_t bytes) override {
        return std::make_unique<LoopbackMr>(fabric_, addr, bytes, true);
    }
    std::unique_ptr<QueuePair> create_qp(int send_depth, int recv_depth) override {
        return std::make_unique<LoopbackQp>(fabric_, send_depth, recv_depth);
    }
    std::uint8_t active_mtu() const override { return 5; }

private:
    std::string name_;
    std::shared_ptr<Fabric> fabric_;
};

}  // namespace

std::shared_ptr<VerbsDevice> make_loopback_device(const std::string& name) {
    return std::make_shared<LoopbackDevice>(name);
}

}  // namespace nano_nccl::rdma
