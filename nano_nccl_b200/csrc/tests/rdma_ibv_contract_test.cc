// The libibverbs provider against a fake function table (no HCA, no libibverbs): what it programs into the
// queue pair and what it sends down the data path.
//
// Parity: the reference guards the same facts with source-text tests (tests/rdma_*_static.py: sq_sig_all = 0,
// selective signalling, inline CTS) and programs them in src/transport/rdma/rdma_qp.cc:93-195 (RC queue pair,
// one completion queue for sends and receives, max_inline_data = 64, INIT -> RTR with the smaller path MTU, a
// GRH on RoCE, min_rnr_timer 12 -> RTS with timeout 14 and retry 7).  Here the provider itself runs and the
// fake records the attribute structs it is handed.
#include "transport/rdma/verbs_ibv.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

using namespace nano_nccl::rdma;

#define CHECK(cond)                                                                        \
    do {                                                                                   \
        if (!(cond)) {                                                                     \
            std::fprintf(stderr, "%s:%d: check failed: %s\n", __FILE__, __LINE__, #cond); \
            std::exit(1);                                                                  \
        }                                                                                  \
    } while (0)

namespace {

struct Recorded {
    ibv_qp_init_attr init{};
    std::vector<std::pair<ibv_qp_attr, int>> modifies;
    std::vector<ibv_send_wr> sends;
    std::vector<ibv_sge> send_sges;
    std::vector<ibv_recv_wr> recvs;
    int cq_depth = 0;
    int reg_access = 0;
    int destroyed_qp = 0, destroyed_cq = 0, dealloc_pd = 0, closed = 0, dereg = 0;
    std::vector<ibv_wc> pending;
} rec;

ibv_context fake_context{};
ibv_cq fake_cq{&fake_context};
ibv_qp fake_qp{};
ibv_mr fake_mr{};
int fake_device_token = 0, fake_pd_token = 0;

int fake_post_send(ibv_qp*, ibv_send_wr* wr, ibv_send_wr**) {
    rec.sends.push_back(*wr);
    rec.send_sges.push_back(wr->num_sge > 0 ? wr->sg_list[0] : ibv_sge{});
    return 0;
}
int fake_post_recv(ibv_qp*, ibv_recv_wr* wr, ibv_recv_wr**) {
    rec.recvs.push_back(*wr);
    return 0;
}
int fake_poll_cq(ibv_cq*, int n, ibv_wc* out) {
    int k = 0;
    while (k < n && !rec.pending.empty()) {
        out[k++] = rec.pending.front();
        rec.pending.erase(rec.pending.begin());
    }
    return k;
}

IbvApi make_fake_api() {
    IbvApi a;
    a.get_device_list = [](int* count) -> ibv_device** {
        static ibv_device* list[2] = {reinterpret_cast<ibv_device*>(&fake_device_token), nullptr};
        *count = 1;
        return list;
    };
    a.free_device_list = [](ibv_device**) {};
    a.get_device_name = [](ibv_device*) -> const char* { return "fake0"; };
    a.open_device = [](ibv_device*) -> ibv_context* { return &fake_context; };
    a.close_device = [](ibv_context*) { ++rec.closed; return 0; };
    a.query_port = [](ibv_context*, std::uint8_t, ibv_port_attr* p) {
        p->state = IBV_PORT_ACTIVE;
        p->active_mtu = IBV_MTU_4096;
        p->lid = 0;
        return 0;
    };
    a.query_gid = [](ibv_context*, std::uint8_t, int, ibv_gid* g) {
        for (int i = 0; i < 16; ++i) g->raw[i] = static_cast<std::uint8_t>(0xa0 + i);
        return 0;
    };
    a.alloc_pd = [](ibv_context*) -> ibv_pd* { return reinterpret_cast<ibv_pd*>(&fake_pd_token); };
    a.dealloc_pd = [](ibv_pd*) { ++rec.dealloc_pd; return 0; };
    a.reg_mr = [](ibv_pd*, void* addr, std::size_t len, int access) -> ibv_mr* {
        rec.reg_access = access;
        fake_mr.addr = addr;
        fake_mr.length = len;
        fake_mr.lkey = 0x1111;
        fake_mr.rkey = 0x2222;
        return &fake_mr;
    };
    a.dereg_mr = [](ibv_mr*) { ++rec.dereg; return 0; };
    a.create_cq = [](ibv_context*, int cqe, void*, ibv_comp_channel*, int) -> ibv_cq* {
        rec.cq_depth = cqe;
        return &fake_cq;
    };
    a.destroy_cq = [](ibv_cq*) { ++rec.destroyed_cq; return 0; };
    a.create_qp = [](ibv_pd*, ibv_qp_init_attr* init) -> ibv_qp* {
        rec.init = *init;
        fake_qp.context = &fake_context;
        fake_qp.qp_num = 77;
        return &fake_qp;
    };
    a.modify_qp = [](ibv_qp*, ibv_qp_attr* attr, int mask) {
        rec.modifies.emplace_back(*attr, mask);
        return 0;
    };
    a.destroy_qp = [](ibv_qp*) { ++rec.destroyed_qp; return 0; };
    a.wc_status_str = [](ibv_wc_status) -> const char* { return "fake failure"; };
    return a;
}

}  // namespace

int main() {
    fake_context.ops.post_send = fake_post_send;
    fake_context.ops.post_recv = fake_post_recv;
    fake_context.ops.poll_cq = fake_poll_cq;
    const IbvApi api = make_fake_api();
    HcaChoice choice;
    choice.hca = "fake0";
    choice.port = 1;
    choice.gid_index = 3;
    choice.roce = true;
    {
        auto device = open_ibverbs_device_with(api, choice);
        CHECK(device != nullptr && device->name() == "fake0" && device->active_mtu() == IBV_MTU_4096);

        // --- queue pair creation: RC, one CQ for both directions, unsignalled by default, 64 inline bytes
        auto qp = device->create_qp(/*send_depth=*/8, /*recv_depth=*/16);
        CHECK(rec.cq_depth == 24);
        CHECK(rec.init.qp_type == IBV_QPT_RC && rec.init.sq_sig_all == 0);
        CHECK(rec.init.send_cq == &fake_cq && rec.init.recv_cq == &fake_cq);
        CHECK(rec.init.cap.max_send_wr == 8 && rec.init.cap.max_recv_wr == 16);
        CHECK(rec.init.cap.max_send_sge == 1 && rec.init.cap.max_recv_sge == 1 && rec.init.cap.max_inline_data == 64);
        CHECK(qp->max_inline() == 64);
        // --- RESET -> INIT at creation, so receives can be posted before the peer is known
        CHECK(rec.modifies.size() == 1);
        CHECK(rec.modifies[0].first.qp_state == IBV_QPS_INIT && rec.modifies[0].first.port_num == 1);
        CHECK(rec.modifies[0].second == (IBV_QP_STATE | IBV_QP_PKEY_INDEX | IBV_QP_PORT | IBV_QP_ACCESS_FLAGS));
        CHECK(rec.modifies[0].first.qp_access_flags == (IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE | IBV_ACCESS_REMOTE_READ));

        RdmaPeerInfo local{};
        qp->fill_local_info(&local);
        CHECK(local.qp_num == 77 && local.gid_index == 3 && local.path_mtu == IBV_MTU_4096 && local.gid[0] == 0xa0 && local.gid[15] == 0xaf);
        CHECK(local.psn <= 0xffffffu);

        // --- INIT -> RTR -> RTS against a peer with a smaller MTU
        RdmaPeerInfo peer{};
        peer.qp_num = 4242;
        peer.psn = 0x123456;
        peer.lid = 0;
        peer.path_mtu = IBV_MTU_1024;
        for (int i = 0; i < 16; ++i) peer.gid[i] = static_cast<std::uint8_t>(i + 1);
        qp->connect(peer);
        CHECK(rec.modifies.size() == 3);
        const ibv_qp_attr& rtr = rec.modifies[1].first;
        CHECK(rtr.qp_state == IBV_QPS_RTR && rtr.path_mtu == IBV_MTU_1024 && rtr.dest_qp_num == 4242 && rtr.rq_psn == 0x123456);
        CHECK(rtr.max_dest_rd_atomic == 1 && rtr.min_rnr_timer == 12);
        CHECK(rtr.ah_attr.is_global == 1 && rtr.ah_attr.port_num == 1 && rtr.ah_attr.grh.sgid_index == 3 && rtr.ah_attr.grh.hop_limit == 64);
        CHECK(std::memcmp(rtr.ah_attr.grh.dgid.raw, peer.gid, 16) == 0);
        CHECK(rec.modifies[1].second == (IBV_QP_STATE | IBV_QP_AV | IBV_QP_PATH_MTU | IBV_QP_DEST_QPN | IBV_QP_RQ_PSN |
                                         IBV_QP_MAX_DEST_RD_ATOMIC | IBV_QP_MIN_RNR_TIMER));
        const ibv_qp_attr& rts = rec.modifies[2].first;
        CHECK(rts.qp_state == IBV_QPS_RTS && rts.timeout == 14 && rts.retry_cnt == 7 && rts.rnr_retry == 7 && rts.max_rd_atomic == 1);
        CHECK(rts.sq_psn == local.psn);
        CHECK(rec.modifies[2].second == (IBV_QP_STATE | IBV_QP_TIMEOUT | IBV_QP_RETRY_CNT | IBV_QP_RNR_RETRY | IBV_QP_SQ_PSN |
                                         IBV_QP_MAX_QP_RD_ATOMIC));

        // --- data path: flags, immediate data, inline only within the limit, zero-length work requests carry no SGE
        alignas(16) static char buffer[4096];
        auto mr = device->register_host(buffer, sizeof(buffer));
        CHECK(rec.reg_access == (IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE | IBV_ACCESS_REMOTE_READ));
        CHECK(mr->lkey() == 0x1111 && mr->rkey() == 0x2222 && !mr->is_device_memory() && !mr->uses_dmabuf());
        qp->post_send(1, Sge{buffer, 256, mr->lkey()}, /*signaled=*/false, /*inline=*/false);
        CHECK(rec.sends.back().opcode == IBV_WR_SEND && rec.sends.back().send_flags == 0 && rec.sends.back().num_sge == 1);
        CHECK(rec.send_sges.back().length == 256 && rec.send_sges.back().lkey == 0x1111);
        qp->post_write(2, Sge{buffer, 32, mr->lkey()}, 0xabc000, 0x9999, /*signaled=*/true, /*inline=*/true);
        CHECK(rec.sends.back().opcode == IBV_WR_RDMA_WRITE && rec.sends.back().send_flags == (IBV_SEND_SIGNALED | IBV_SEND_INLINE));
        CHECK(rec.sends.back().wr.rdma.remote_addr == 0xabc000 && rec.sends.back().wr.rdma.rkey == 0x9999);
        qp->post_write(3, Sge{buffer, 65, mr->lkey()}, 0xabc000, 0x9999, false, /*inline=*/true);
        CHECK(rec.sends.back().send_flags == 0);  // 65 bytes exceed the inline limit
        qp->post_write_imm(4, Sge{buffer, 0, mr->lkey()}, 0xabc000, 0x9999, /*imm_be=*/0x01020304u, true);
        CHECK(rec.sends.back().opcode == IBV_WR_RDMA_WRITE_WITH_IMM && rec.sends.back().imm_data == 0x01020304u);
        CHECK(rec.sends.back().num_sge == 0 && rec.sends.back().sg_list == nullptr && rec.sends.back().wr_id == 4);
        qp->post_recv(9, Sge{buffer, 1, mr->lkey()});
        CHECK(rec.recvs.back().wr_id == 9 && rec.recvs.back().num_sge == 1);

        // --- completions: opcode mapping, immediate kept big-endian, a failed completion carries its text
        ibv_wc ok{};
        ok.wr_id = 4;
        ok.status = IBV_WC_SUCCESS;
        ok.opcode = IBV_WC_RECV_RDMA_WITH_IMM;
        ok.byte_len = 0;
        ok.imm_data = 0x01020304u;
        ibv_wc bad{};
        bad.wr_id = 5;
        bad.status = static_cast<ibv_wc_status>(12);
        bad.vendor_err = 129;
        rec.pending = {ok, bad};
        WorkCompletion wc[4];
        CHECK(qp->poll(wc, 4) == 2);
        CHECK(wc[0].ok && wc[0].opcode == WcOpcode::RecvImm && wc[0].imm_be == 0x01020304u && wc[0].wr_id == 4);
        CHECK(!wc[1].ok && wc[1].error.find("fake failure") != std::string::npos && wc[1].error.find("129") != std::string::npos);
        CHECK(qp->poll(wc, 4) == 0);
    }
    // everything was released, in dependency order: region and queue pair before the protection domain and the context
    CHECK(rec.dereg == 1 && rec.destroyed_qp == 1 && rec.destroyed_cq == 1 && rec.dealloc_pd == 1 && rec.closed == 1);

    // the real binding on a machine without RDMA: a clean answer, no crash
    std::string why;
    if (load_ibverbs(&why) == nullptr) {
        CHECK(why.find("libibverbs") != std::string::npos);
        RdmaConfig cfg;
        std::string reason;
        CHECK(open_ibverbs_device(cfg, &reason) == nullptr && reason.find("no RDMA device") != std::string::npos);
    }
    std::printf("rdma_ibv_contract_test ok\n");
    return 0;
}
