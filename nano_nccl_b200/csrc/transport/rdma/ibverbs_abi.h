// Declarations of exactly the part of the libibverbs ABI that the verbs provider uses, so that the provider
// is compiled in every build, with or without <infiniband/verbs.h> on the build machine, and binds to
// libibverbs.so.1 at run time with dlopen (as the topology code does with the management library).
//
// The layouts and values restate the stable "IBVERBS_1.1" ABI of rdma-core's public header
// (infiniband/verbs.h).  Objects that the library allocates (context, protection domain, completion queue,
// queue pair, memory region) are declared only as far as this code reads them; they are never created or
// copied here.  Work requests, completions and attribute structs are passed by address and therefore declared
// in full, with their sizes pinned by static_asserts.
//
// Entry points that the real header implements as inline functions over the context's operation table
// (post_send, post_recv, poll_cq) are reached the same way here: through `ibv_context::ops`.
//
// The reference includes <infiniband/verbs.h> directly (src/transport/rdma/rdma_qp.cc, rdma_endpoint.cc,
// rdma_gdr.cc); it therefore builds its RDMA transport only where that header is installed.
#pragma once

#include <pthread.h>

#include <cstddef>
#include <cstdint>

extern "C" {

struct ibv_device;
struct ibv_pd;
struct ibv_srq;
struct ibv_ah;
struct ibv_mw;
struct ibv_comp_channel;
struct ibv_qp;
struct ibv_cq;
struct ibv_context;

enum ibv_qp_type : int { IBV_QPT_RC = 2 };
enum ibv_qp_state : int { IBV_QPS_RESET = 0, IBV_QPS_INIT = 1, IBV_QPS_RTR = 2, IBV_QPS_RTS = 3 };
enum ibv_mtu : int { IBV_MTU_256 = 1, IBV_MTU_512 = 2, IBV_MTU_1024 = 3, IBV_MTU_2048 = 4, IBV_MTU_4096 = 5 };
enum ibv_port_state : int { IBV_PORT_DOWN = 1, IBV_PORT_INIT = 2, IBV_PORT_ARMED = 3, IBV_PORT_ACTIVE = 4 };
enum ibv_mig_state : int { IBV_MIG_MIGRATED = 0 };
enum ibv_access_flags : int { IBV_ACCESS_LOCAL_WRITE = 1, IBV_ACCESS_REMOTE_WRITE = 2, IBV_ACCESS_REMOTE_READ = 4 };
enum ibv_wr_opcode : int { IBV_WR_RDMA_WRITE = 0, IBV_WR_RDMA_WRITE_WITH_IMM = 1, IBV_WR_SEND = 2 };
enum ibv_send_flags : int { IBV_SEND_FENCE = 1, IBV_SEND_SIGNALED = 2, IBV_SEND_SOLICITED = 4, IBV_SEND_INLINE = 8 };
enum ibv_wc_status : int { IBV_WC_SUCCESS = 0 };
enum ibv_wc_opcode : int { IBV_WC_SEND = 0, IBV_WC_RDMA_WRITE = 1, IBV_WC_RECV = 128, IBV_WC_RECV_RDMA_WITH_IMM = 129 };
enum ibv_qp_attr_mask : int {
    IBV_QP_STATE = 1 << 0, IBV_QP_ACCESS_FLAGS = 1 << 3, IBV_QP_PKEY_INDEX = 1 << 4, IBV_QP_PORT = 1 << 5,
    IBV_QP_AV = 1 << 7, IBV_QP_PATH_MTU = 1 << 8, IBV_QP_TIMEOUT = 1 << 9, IBV_QP_RETRY_CNT = 1 << 10,
    IBV_QP_RNR_RETRY = 1 << 11, IBV_QP_RQ_PSN = 1 << 12, IBV_QP_MAX_QP_RD_ATOMIC = 1 << 13,
    IBV_QP_MIN_RNR_TIMER = 1 << 15, IBV_QP_SQ_PSN = 1 << 16, IBV_QP_MAX_DEST_RD_ATOMIC = 1 << 17,
    IBV_QP_DEST_QPN = 1 << 20,
};

struct ibv_gid_global { std::uint64_t subnet_prefix; std::uint64_t interface_id; };
union ibv_gid {
    std::uint8_t raw[16];
    ibv_gid_global global;
};

struct ibv_sge { std::uint64_t addr; std::uint32_t length; std::uint32_t lkey; };

struct ibv_mw_bind_info { void* mr; std::uint64_t addr; std::uint64_t length; unsigned int mw_access_flags; };
struct ibv_send_wr_bind_mw { ibv_mw* mw; std::uint32_t rkey; ibv_mw_bind_info bind_info; };
struct ibv_send_wr_tso { void* hdr; std::uint16_t hdr_sz; std::uint16_t mss; };
struct ibv_send_wr_rdma { std::uint64_t remote_addr; std::uint32_t rkey; };
struct ibv_send_wr_atomic { std::uint64_t remote_addr; std::uint64_t compare_add; std::uint64_t swap; std::uint32_t rkey; };
struct ibv_send_wr_ud { ibv_ah* ah; std::uint32_t remote_qpn; std::uint32_t remote_qkey; };

struct ibv_send_wr {
    std::uint64_t wr_id;
    ibv_send_wr* next;
    ibv_sge* sg_list;
    int num_sge;
    ibv_wr_opcode opcode;
    unsigned int send_flags;
    std::uint32_t imm_data;  // big-endian; shares its place with invalidate_rkey
    union {
        ibv_send_wr_rdma rdma;
        ibv_send_wr_atomic atomic;
        ibv_send_wr_ud ud;
    } wr;
    std::uint32_t xrc_remote_srqn;
    union {
        ibv_send_wr_bind_mw bind_mw;
        ibv_send_wr_tso tso;
    } tail;
};

struct ibv_recv_wr { std::uint64_t wr_id; ibv_recv_wr* next; ibv_sge* sg_list; int num_sge; };

struct ibv_wc {
    std::uint64_t wr_id;
    ibv_wc_status status;
    ibv_wc_opcode opcode;
    std::uint32_t vendor_err;
    std::uint32_t byte_len;
    std::uint32_t imm_data;  // big-endian; shares its place with invalidated_rkey
    std::uint32_t qp_num;
    std::uint32_t src_qp;
    unsigned int wc_flags;
    std::uint16_t pkey_index;
    std::uint16_t slid;
    std::uint8_t sl;
    std::uint8_t dlid_path_bits;
};

struct ibv_qp_cap {
    std::uint32_t max_send_wr, max_recv_wr, max_send_sge, max_recv_sge, max_inline_data;
};

struct ibv_qp_init_attr {
    void* qp_context;
    ibv_cq* send_cq;
    ibv_cq* recv_cq;
    ibv_srq* srq;
    ibv_qp_cap cap;
    ibv_qp_type qp_type;
    int sq_sig_all;
};

struct ibv_global_route {
    ibv_gid dgid;
    std::uint32_t flow_label;
    std::uint8_t sgid_index, hop_limit, traffic_class;
};

struct ibv_ah_attr {
    ibv_global_route grh;
    std::uint16_t dlid;
    std::uint8_t sl, src_path_bits, static_rate, is_global, port_num;
};

struct ibv_qp_attr {
    ibv_qp_state qp_state, cur_qp_state;
    ibv_mtu path_mtu;
    ibv_mig_state path_mig_state;
    std::uint32_t qkey, rq_psn, sq_psn, dest_qp_num;
    unsigned int qp_access_flags;
    ibv_qp_cap cap;
    ibv_ah_attr ah_attr, alt_ah_attr;
    std::uint16_t pkey_index, alt_pkey_index;
    std::uint8_t en_sqd_async_notify, sq_draining, max_rd_atomic, max_dest_rd_atomic, min_rnr_timer, port_num, timeout,
        retry_cnt, rnr_retry, alt_port_num, alt_timeout;
    std::uint32_t rate_limit;
};

// The exported ibv_query_port fills the original (shorter) form of this struct; the extra room at the end
// covers every later extension of it.
struct ibv_port_attr {
    ibv_port_state state;
    ibv_mtu max_mtu, active_mtu;
    int gid_tbl_len;
    std::uint32_t port_cap_flags, max_msg_sz, bad_pkey_cntr, qkey_viol_cntr;
    std::uint16_t pkey_tbl_len, lid, sm_lid;
    std::uint8_t lmc, max_vl_num, sm_sl, subnet_timeout, init_type_reply, active_width, active_speed, phys_state, link_layer, flags;
    std::uint16_t port_cap_flags2;
    std::uint32_t active_speed_ex;
    std::uint8_t room_for_extensions[64];
};

struct ibv_mr {
    ibv_context* context;
    ibv_pd* pd;
    void* addr;
    std::size_t length;
    std::uint32_t handle, lkey, rkey;
};

// The operation table at the head of every context.  Only the three data-path entries are called here; the
// other slots keep the table's shape.
struct ibv_context_ops {
    void* compat_head[7];                                       // query_device .. dereg_mr
    void* alloc_mw; void* bind_mw; void* dealloc_mw;
    void* compat_create_cq;
    int (*poll_cq)(ibv_cq* cq, int num_entries, ibv_wc* wc);
    void* req_notify_cq;
    void* compat_cq[3];                                         // cq_event, resize_cq, destroy_cq
    void* compat_srq[4];                                        // create, modify, query, destroy
    void* post_srq_recv;
    void* compat_qp[4];                                         // create, query, modify, destroy
    int (*post_send)(ibv_qp* qp, ibv_send_wr* wr, ibv_send_wr** bad_wr);
    int (*post_recv)(ibv_qp* qp, ibv_recv_wr* wr, ibv_recv_wr** bad_wr);
    void* compat_tail[5];                                       // create_ah, destroy_ah, attach / detach mcast, async_event
};

struct ibv_context {
    ibv_device* device;
    ibv_context_ops ops;
    int cmd_fd, async_fd, num_comp_vectors;
    pthread_mutex_t mutex;
    void* abi_compat;
};

// Heads of two library-owned objects, as far as they are read here.
struct ibv_cq { ibv_context* context; };
struct ibv_qp {
    ibv_context* context;
    void* qp_context;
    ibv_pd* pd;
    ibv_cq* send_cq;
    ibv_cq* recv_cq;
    ibv_srq* srq;
    std::uint32_t handle, qp_num;
};

}  // extern "C"

static_assert(sizeof(ibv_sge) == 16 && sizeof(ibv_recv_wr) == 32, "verbs ABI: scatter / receive request layout");
static_assert(sizeof(ibv_send_wr) == 128 && offsetof(ibv_send_wr, wr) == 40 && offsetof(ibv_send_wr, imm_data) == 36,
              "verbs ABI: send request layout");
static_assert(sizeof(ibv_wc) == 48 && offsetof(ibv_wc, byte_len) == 20 && offsetof(ibv_wc, imm_data) == 24, "verbs ABI: completion layout");
static_assert(sizeof(ibv_qp_init_attr) == 64 && offsetof(ibv_qp_init_attr, sq_sig_all) == 56, "verbs ABI: queue pair creation layout");
static_assert(sizeof(ibv_ah_attr) == 32 && offsetof(ibv_ah_attr, dlid) == 24, "verbs ABI: address vector layout");
static_assert(sizeof(ibv_qp_attr) == 144 && offsetof(ibv_qp_attr, ah_attr) == 56 && offsetof(ibv_qp_attr, max_rd_atomic) == 126 &&
                  offsetof(ibv_qp_attr, rate_limit) == 136, "verbs ABI: queue pair attribute layout");
static_assert(offsetof(ibv_port_attr, lid) == 34 && offsetof(ibv_port_attr, active_mtu) == 8, "verbs ABI: port attribute layout");
static_assert(sizeof(ibv_context_ops) == 32 * sizeof(void*) && offsetof(ibv_context_ops, poll_cq) == 11 * sizeof(void*) &&
                  offsetof(ibv_context_ops, post_send) == 25 * sizeof(void*) && offsetof(ibv_context_ops, post_recv) == 26 * sizeof(void*),
              "verbs ABI: operation table layout");
static_assert(offsetof(ibv_mr, lkey) == 36 && offsetof(ibv_qp, qp_num) == 52, "verbs ABI: memory region / queue pair heads");

namespace nano_nccl::rdma {

// The exported functions of libibverbs that the provider calls, resolved once at run time.
struct IbvApi {
    ibv_device** (*get_device_list)(int* count) = nullptr;
    void (*free_device_list)(ibv_device** list) = nullptr;
    const char* (*get_device_name)(ibv_device* device) = nullptr;
    ibv_context* (*open_device)(ibv_device* device) = nullptr;
    int (*close_device)(ibv_context* context) = nullptr;
    int (*query_port)(ibv_context* context, std::uint8_t port, ibv_port_attr* attr) = nullptr;
    int (*query_gid)(ibv_context* context, std::uint8_t port, int index, ibv_gid* gid) = nullptr;
    ibv_pd* (*alloc_pd)(ibv_context* context) = nullptr;
    int (*dealloc_pd)(ibv_pd* pd) = nullptr;
    ibv_mr* (*reg_mr)(ibv_pd* pd, void* addr, std::size_t length, int access) = nullptr;
    ibv_mr* (*reg_dmabuf_mr)(ibv_pd* pd, std::uint64_t offset, std::size_t length, std::uint64_t iova, int fd, int access) = nullptr;  // optional
    int (*dereg_mr)(ibv_mr* mr) = nullptr;
    ibv_cq* (*create_cq)(ibv_context* context, int cqe, void* cq_context, ibv_comp_channel* channel, int comp_vector) = nullptr;
    int (*destroy_cq)(ibv_cq* cq) = nullptr;
    ibv_qp* (*create_qp)(ibv_pd* pd, ibv_qp_init_attr* attr) = nullptr;
    int (*modify_qp)(ibv_qp* qp, ibv_qp_attr* attr, int mask) = nullptr;
    int (*destroy_qp)(ibv_qp* qp) = nullptr;
    const char* (*wc_status_str)(ibv_wc_status status) = nullptr;
};

}  // namespace nano_nccl::rdma
