// libibverbs provider of the verbs interface.  Always compiled: the verbs ABI it needs is declared in
// ibverbs_abi.h and the library is bound at run time with dlopen, so a machine without RDMA hardware or
// without libibverbs gets a clean "no RDMA device" answer from open_ibverbs_device() instead of a build
// that lacks the provider.
//
// Parity: reference src/transport/rdma/rdma_qp.cc:93-195 (RC queue pair with one completion queue
// shared by sends and receives, sq_sig_all = 0, max_inline_data = 64; INIT -> RTR with
// path_mtu = min(local, remote), a GRH on RoCE and min_rnr_timer 12 -> RTS with timeout 14 and
// retry 7), rdma_endpoint.cc:164-236 (device selection, port 1 ACTIVE) and rdma_gdr.cc:28-64,
// 197-217 (GPU memory: CU_POINTER_ATTRIBUTE_SYNC_MEMOPS, then a dma-buf registration, then the
// peer-memory registration; never a silent fall back to host memory).
#include "transport/rdma/verbs_ibv.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <mutex>
#include <random>
#include <stdexcept>

namespace nano_nccl::rdma {
namespace {

constexpr int kAccess = IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE | IBV_ACCESS_REMOTE_READ;
constexpr std::uint32_t kMaxInline = 64;

[[noreturn]] void fail(const std::string& what) { throw std::runtime_error("RDMA transport: " + what); }

template <typename Fn>
Fn driver_entry(const char* name) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult status = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &status) != cudaSuccess ||
        status != cudaDriverEntryPointSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return reinterpret_cast<Fn>(fn);
}

class IbvMemoryRegion final : public MemoryRegion {
public:
    IbvMemoryRegion(const IbvApi& api, ibv_mr* mr, void* addr, std::size_t bytes, bool device, int dmabuf_fd)
        : api_(api), mr_(mr), addr_(addr), bytes_(bytes), device_(device), dmabuf_fd_(dmabuf_fd) {}
    ~IbvMemoryRegion() override {
        if (mr_ != nullptr) api_.dereg_mr(mr_);
        if (dmabuf_fd_ >= 0) close(dmabuf_fd_);
    }
    std::uint32_t lkey() const override { return mr_->lkey; }
    std::uint32_t rkey() const override { return mr_->rkey; }
    void* addr() const override { return addr_; }
    std::size_t length() const override { return bytes_; }
    bool is_device_memory() const override { return device_; }
    bool uses_dmabuf() const override { return dmabuf_fd_ >= 0; }

private:
    const IbvApi& api_;
    ibv_mr* mr_;
    void* addr_;
    std::size_t bytes_;
    bool device_;
    int dmabuf_fd_;
};

struct Shared {
    explicit Shared(const IbvApi& a) : api(a) {}
    const IbvApi& api;
    ibv_context* context = nullptr;
    ibv_pd* pd = nullptr;
    ibv_port_attr port{};
    ibv_gid gid{};
    HcaChoice choice;
    ~Shared() {
        if (pd != nullptr) api.dealloc_pd(pd);
        if (context != nullptr) api.close_device(context);
    }
};

class IbvQueuePair final : public QueuePair {
public:
    IbvQueuePair(std::shared_ptr<Shared> shared, int send_depth, int recv_depth) : shared_(std::move(shared)) {
        cq_ = api().create_cq(shared_->context, send_depth + recv_depth, nullptr, nullptr, 0);
        if (cq_ == nullptr) fail("ibv_create_cq failed");
        ibv_qp_init_attr init{};
        init.send_cq = cq_;
        init.recv_cq = cq_;
        init.qp_type = IBV_QPT_RC;
        init.sq_sig_all = 0;
        init.cap.max_send_wr = static_cast<std::uint32_t>(send_depth);
        init.cap.max_recv_wr = static_cast<std::uint32_t>(recv_depth);
        init.cap.max_send_sge = 1;
        init.cap.max_recv_sge = 1;
        init.cap.max_inline_data = kMaxInline;
        qp_ = api().create_qp(shared_->pd, &init);
        if (qp_ == nullptr) {
            api().destroy_cq(cq_);
            cq_ = nullptr;
            fail("ibv_create_qp failed");
        }
        max_inline_ = init.cap.max_inline_data;
        std::random_device rd;
        psn_ = rd() & 0xffffffu;
        // INIT right away: receive work requests may be posted before the peer is known.
        ibv_qp_attr attr{};
        attr.qp_state = IBV_QPS_INIT;
        attr.pkey_index = 0;
        attr.port_num = static_cast<std::uint8_t>(shared_->choice.port);
        attr.qp_access_flags = kAccess;
        if (api().modify_qp(qp_, &attr, IBV_QP_STATE | IBV_QP_PKEY_INDEX | IBV_QP_PORT | IBV_QP_ACCESS_FLAGS) != 0) {
            destroy();
            fail("queue pair RESET -> INIT failed");
        }
    }
    ~IbvQueuePair() override { destroy(); }

    void post_send(std::uint64_t wr_id, const Sge& sge, bool signaled, bool inline_data) override {
        post(wr_id, sge, IBV_WR_SEND, 0, 0, 0, signaled, inline_data);
    }
    void post_write(std::uint64_t wr_id, const Sge& sge, std::uint64_t raddr, std::uint32_t rkey, bool signaled,
                    bool inline_data) override {
        post(wr_id, sge, IBV_WR_RDMA_WRITE, raddr, rkey, 0, signaled, inline_data);
    }
    void post_write_imm(std::uint64_t wr_id, const Sge& sge, std::uint64_t raddr, std::uint32_t rkey,
                        std::uint32_t imm_be, bool signaled) override {
        post(wr_id, sge, IBV_WR_RDMA_WRITE_WITH_IMM, raddr, rkey, imm_be, signaled, false);
    }
    void post_recv(std::uint64_t wr_id, const Sge& sge) override {
        ibv_sge s{};
        s.addr = reinterpret_cast<std::uint64_t>(sge.addr);
        s.length = sge.length;
        s.lkey = sge.lkey;
        ibv_recv_wr wr{};
        wr.wr_id = wr_id;
        wr.sg_list = &s;
        wr.num_sge = 1;
        ibv_recv_wr* bad = nullptr;
        if (qp_->context->ops.post_recv(qp_, &wr, &bad) != 0) fail("ibv_post_recv failed");
    }
    int poll(WorkCompletion* out, int max) override {
        constexpr int kBatch = 16;
        ibv_wc wc[kBatch];
        const int n = cq_->context->ops.poll_cq(cq_, std::min(max, kBatch), wc);
        if (n < 0) fail("ibv_poll_cq failed");
        for (int i = 0; i < n; ++i) {
            WorkCompletion& c = out[i];
            c = WorkCompletion{};
            c.wr_id = wc[i].wr_id;
            c.ok = wc[i].status == IBV_WC_SUCCESS;
            if (!c.ok) {
                c.error = std::string(api().wc_status_str(wc[i].status)) + " (vendor error " + std::to_string(wc[i].vendor_err) + ")";
                continue;  // the opcode of a failed completion is not defined
            }
            switch (wc[i].opcode) {
                case IBV_WC_SEND: c.opcode = WcOpcode::Send; break;
                case IBV_WC_RDMA_WRITE: c.opcode = WcOpcode::Write; break;
                case IBV_WC_RECV: c.opcode = WcOpcode::Recv; break;
                case IBV_WC_RECV_RDMA_WITH_IMM: c.opcode = WcOpcode::RecvImm; break;
                default: c.ok = false; c.error = "unexpected completion opcode " + std::to_string(wc[i].opcode); break;
            }
            c.byte_len = wc[i].byte_len;
            c.imm_be = wc[i].imm_data;  // kept big-endian, as on the wire
        }
        return n;
    }
    std::uint32_t max_inline() const override { return max_inline_; }
    void fill_local_info(RdmaPeerInfo* info) const override {
        info->qp_num = qp_->qp_num;
        info->psn = psn_;
        info->lid = shared_->port.lid;
        info->gid_index = static_cast<std::uint8_t>(shared_->choice.gid_index);
        info->path_mtu = static_cast<std::uint8_t>(shared_->port.active_mtu);
        std::memcpy(info->gid, shared_->gid.raw, 16);
    }
    void connect(const RdmaPeerInfo& peer) override {
        ibv_qp_attr attr{};
        attr.qp_state = IBV_QPS_RTR;
        attr.path_mtu = static_cast<ibv_mtu>(negotiate_path_mtu(static_cast<std::uint8_t>(shared_->port.active_mtu), peer.path_mtu));
        attr.dest_qp_num = peer.qp_num;
        attr.rq_psn = peer.psn;
        attr.max_dest_rd_atomic = 1;
        attr.min_rnr_timer = 12;
        attr.ah_attr.dlid = peer.lid;
        attr.ah_attr.sl = 0;
        attr.ah_attr.src_path_bits = 0;
        attr.ah_attr.port_num = static_cast<std::uint8_t>(shared_->choice.port);
        if (shared_->choice.roce || peer.lid == 0) {
            attr.ah_attr.is_global = 1;
            std::memcpy(attr.ah_attr.grh.dgid.raw, peer.gid, 16);
            attr.ah_attr.grh.sgid_index = static_cast<std::uint8_t>(shared_->choice.gid_index);
            attr.ah_attr.grh.hop_limit = 64;
            attr.ah_attr.grh.traffic_class = 0;
            attr.ah_attr.grh.flow_label = 0;
        }
        if (api().modify_qp(qp_, &attr,
                          IBV_QP_STATE | IBV_QP_AV | IBV_QP_PATH_MTU | IBV_QP_DEST_QPN | IBV_QP_RQ_PSN |
                              IBV_QP_MAX_DEST_RD_ATOMIC | IBV_QP_MIN_RNR_TIMER) != 0) {
            fail("queue pair INIT -> RTR failed");
        }
        ibv_qp_attr rts{};
        rts.qp_state = IBV_QPS_RTS;
        rts.timeout = 14;
        rts.retry_cnt = 7;
        rts.rnr_retry = 7;
        rts.sq_psn = psn_;
        rts.max_rd_atomic = 1;
        if (api().modify_qp(qp_, &rts,
                          IBV_QP_STATE | IBV_QP_TIMEOUT | IBV_QP_RETRY_CNT | IBV_QP_RNR_RETRY | IBV_QP_SQ_PSN |
                              IBV_QP_MAX_QP_RD_ATOMIC) != 0) {
            fail("queue pair RTR -> RTS failed");
        }
    }

private:
    void post(std::uint64_t wr_id, const Sge& sge, ibv_wr_opcode opcode, std::uint64_t raddr, std::uint32_t rkey,
              std::uint32_t imm_be, bool signaled, bool inline_data) {
        ibv_sge s{};
        s.addr = reinterpret_cast<std::uint64_t>(sge.addr);
        s.length = sge.length;
        s.lkey = sge.lkey;
        ibv_send_wr wr{};
        wr.wr_id = wr_id;
        wr.sg_list = sge.length == 0 ? nullptr : &s;
        wr.num_sge = sge.length == 0 ? 0 : 1;
        wr.opcode = opcode;
        wr.send_flags = (signaled ? IBV_SEND_SIGNALED : 0) |
                        (inline_data && sge.length <= max_inline_ ? IBV_SEND_INLINE : 0);
        wr.imm_data = imm_be;
        if (opcode != IBV_WR_SEND) {
            wr.wr.rdma.remote_addr = raddr;
            wr.wr.rdma.rkey = rkey;
        }
        ibv_send_wr* bad = nullptr;
        if (qp_->context->ops.post_send(qp_, &wr, &bad) != 0) fail("ibv_post_send failed");
    }
    void destroy() {
        if (qp_ != nullptr) api().destroy_qp(qp_);
        if (cq_ != nullptr) api().destroy_cq(cq_);
        qp_ = nullptr;
        cq_ = nullptr;
    }

    const IbvApi& api() const { return shared_->api; }

    std::shared_ptr<Shared> shared_;
    ibv_cq* cq_ = nullptr;
    ibv_qp* qp_ = nullptr;
    std::uint32_t max_inline_ = 0;
    std::uint32_t psn_ = 0;
};

class IbvDevice final : public VerbsDevice {
public:
    explicit IbvDevice(std::shared_ptr<Shared> shared) : shared_(std::move(shared)) {}
    std::string name() const override { return shared_->choice.hca; }
    std::unique_ptr<MemoryRegion> register_host(void* addr, std::size_t bytes) override {
        ibv_mr* mr = shared_->api.reg_mr(shared_->pd, addr, bytes, kAccess);
        if (mr == nullptr) fail("ibv_reg_mr of host memory failed");
        return std::make_unique<IbvMemoryRegion>(shared_->api, mr, addr, bytes, false, -1);
    }
    std::unique_ptr<MemoryRegion> register_device(void* addr, std::size_t bytes) override {
        // Synchronous memory operations on the range, so that a copy into it is complete when the call returns.
        using SetAttr = CUresult (*)(const void*, CUpointer_attribute, CUdeviceptr);
        if (auto set = driver_entry<SetAttr>("cuPointerSetAttribute")) {
            const unsigned int on = 1;
            set(&on, CU_POINTER_ATTRIBUTE_SYNC_MEMOPS, reinterpret_cast<CUdeviceptr>(addr));
        }
        // 1. dma-buf export of the range, registered through ibv_reg_dmabuf_mr (rdma-core 34 or later).
        using GetHandle = CUresult (*)(void*, CUdeviceptr, size_t, CUmemRangeHandleType, unsigned long long);
        auto get_handle = driver_entry<GetHandle>("cuMemGetHandleForAddressRange");
        auto reg_dmabuf = shared_->api.reg_dmabuf_mr;
        if (get_handle != nullptr && reg_dmabuf != nullptr) {
            int fd = -1;
            if (get_handle(&fd, reinterpret_cast<CUdeviceptr>(addr), bytes, CU_MEM_RANGE_HANDLE_TYPE_DMA_BUF_FD, 0) ==
                    CUDA_SUCCESS && fd >= 0) {
                ibv_mr* mr = reg_dmabuf(shared_->pd, 0, bytes, reinterpret_cast<std::uint64_t>(addr), fd, kAccess);
                if (mr != nullptr) return std::make_unique<IbvMemoryRegion>(shared_->api, mr, addr, bytes, true, fd);
                close(fd);
            }
        }
        // 2. the peer-memory path: the HCA driver resolves the GPU address itself.
        ibv_mr* mr = shared_->api.reg_mr(shared_->pd, addr, bytes, kAccess);
        if (mr == nullptr) {
            fail("GPU memory could not be registered (neither dma-buf nor peer memory); GPUDirect was requested "
                 "explicitly, so host staging is not used instead");
        }
        return std::make_unique<IbvMemoryRegion>(shared_->api, mr, addr, bytes, true, -1);
    }
    std::unique_ptr<QueuePair> create_qp(int send_depth, int recv_depth) override {
        return std::make_unique<IbvQueuePair>(shared_, send_depth, recv_depth);
    }
    std::uint8_t active_mtu() const override { return static_cast<std::uint8_t>(shared_->port.active_mtu); }

private:
    std::shared_ptr<Shared> shared_;
};

}  // namespace

const IbvApi* load_ibverbs(std::string* why) {
    static std::once_flag once;
    static IbvApi api;
    static std::string problem;
    static bool ok = false;
    std::call_once(once, [] {
        void* lib = dlopen("libibverbs.so.1", RTLD_NOW | RTLD_GLOBAL);
        if (lib == nullptr) {
            problem = "no RDMA device: libibverbs.so.1 cannot be loaded on this machine";
            return;
        }
        auto bind = [&](auto& slot, const char* name, bool required) {
            slot = reinterpret_cast<std::remove_reference_t<decltype(slot)>>(dlsym(lib, name));
            if (slot == nullptr && required && problem.empty()) problem = std::string("libibverbs.so.1 lacks ") + name;
        };
        bind(api.get_device_list, "ibv_get_device_list", true);
        bind(api.free_device_list, "ibv_free_device_list", true);
        bind(api.get_device_name, "ibv_get_device_name", true);
        bind(api.open_device, "ibv_open_device", true);
        bind(api.close_device, "ibv_close_device", true);
        bind(api.query_port, "ibv_query_port", true);
        bind(api.query_gid, "ibv_query_gid", true);
        bind(api.alloc_pd, "ibv_alloc_pd", true);
        bind(api.dealloc_pd, "ibv_dealloc_pd", true);
        bind(api.reg_mr, "ibv_reg_mr", true);
        bind(api.reg_dmabuf_mr, "ibv_reg_dmabuf_mr", false);  // rdma-core 34 or later
        bind(api.dereg_mr, "ibv_dereg_mr", true);
        bind(api.create_cq, "ibv_create_cq", true);
        bind(api.destroy_cq, "ibv_destroy_cq", true);
        bind(api.create_qp, "ibv_create_qp", true);
        bind(api.modify_qp, "ibv_modify_qp", true);
        bind(api.destroy_qp, "ibv_destroy_qp", true);
        bind(api.wc_status_str, "ibv_wc_status_str", true);
        ok = problem.empty();
    });
    if (!ok) {
        if (why != nullptr) *why = problem;
        return nullptr;
    }
    return &api;
}

std::shared_ptr<VerbsDevice> open_ibverbs_device_with(const IbvApi& api, const HcaChoice& choice) {
    int count = 0;
    ibv_device** list = api.get_device_list(&count);
    if (list == nullptr || count == 0) fail("no RDMA device: ibv_get_device_list found none");
    auto shared = std::make_shared<Shared>(api);
    shared->choice = choice;
    for (int i = 0; i < count && shared->context == nullptr; ++i) {
        if (choice.hca == api.get_device_name(list[i])) shared->context = api.open_device(list[i]);
    }
    api.free_device_list(list);
    if (shared->context == nullptr) fail("ibv_open_device(" + choice.hca + ") failed");
    if (api.query_port(shared->context, static_cast<std::uint8_t>(choice.port), &shared->port) != 0) fail("ibv_query_port failed");
    if (shared->port.state != IBV_PORT_ACTIVE) fail("port " + std::to_string(choice.port) + " of " + choice.hca + " is not ACTIVE");
    if (api.query_gid(shared->context, static_cast<std::uint8_t>(choice.port), choice.gid_index, &shared->gid) != 0) {
        fail("ibv_query_gid(" + std::to_string(choice.gid_index) + ") failed");
    }
    shared->pd = api.alloc_pd(shared->context);
    if (shared->pd == nullptr) fail("ibv_alloc_pd failed");
    return std::make_shared<IbvDevice>(std::move(shared));
}

std::shared_ptr<VerbsDevice> open_ibverbs_device(const RdmaConfig& config, std::string* why) {
    try {
        const IbvApi* api = load_ibverbs(why);
        if (api == nullptr) return nullptr;
        const HcaChoice choice = select_hca(config.ifname, config.gid_index, interface_gids(config.ifname));
        return open_ibverbs_device_with(*api, choice);
    } catch (const std::exception& e) {
        if (why != nullptr) *why = e.what();
        return nullptr;
    }
}

}  // namespace nano_nccl::rdma
