// The slice of the verbs API the RDMA proxies need, behind an interface, with two providers:
// libibverbs (always compiled against in-tree declarations of its ABI, bound with dlopen at run time)
// and an in-process loopback fabric with reliable-connected semantics used by the unit tests
// (in-order delivery, receive WQEs consumed in order, completions in order, immediate data,
// remote-key and bounds checks on RDMA writes).
//
// Parity: the reference programs libibverbs directly (src/transport/rdma/rdma_qp.cc:93-195:
// RC QP, one CQ shared by send and receive, sq_sig_all = 0, max_inline_data = 64; rdma_endpoint.cc:
// 164-236 device selection) and tests on one HCA in loopback (tests/rdma_proxy_test.cc); the
// interface lets the same proxy code run against either.
#pragma once

#include "transport/rdma/rdma_protocol.h"

#include <cstdint>
#include <memory>
#include <string>

namespace nano_nccl::rdma {

enum class WcOpcode { Send, Recv, RecvImm, Write };

struct WorkCompletion {
    std::uint64_t wr_id = 0;
    bool ok = true;
    WcOpcode opcode = WcOpcode::Send;
    std::uint32_t byte_len = 0;   // receives: payload bytes
    std::uint32_t imm_be = 0;     // RecvImm: immediate data, big-endian as on the wire
    std::string error;            // when !ok
};

struct Sge {
    void* addr = nullptr;
    std::uint32_t length = 0;
    std::uint32_t lkey = 0;
};

class MemoryRegion {
public:
    virtual ~MemoryRegion() = default;
    virtual std::uint32_t lkey() const = 0;
    virtual std::uint32_t rkey() const = 0;
    virtual void* addr() const = 0;
    virtual std::size_t length() const = 0;
    virtual bool is_device_memory() const = 0;
    virtual bool uses_dmabuf() const = 0;
};

class QueuePair {
public:
    virtual ~QueuePair() = default;
    // signaled: ask for a send completion.  Unsignaled sends complete silently (RC keeps order,
    // so a later signaled completion retires them too).
    virtual void post_send(std::uint64_t wr_id, const Sge& sge, bool signaled, bool inline_data) = 0;
    virtual void post_write(std::uint64_t wr_id, const Sge& sge, std::uint64_t raddr, std::uint32_t rkey,
                            bool signaled, bool inline_data) = 0;
    virtual void post_write_imm(std::uint64_t wr_id, const Sge& sge, std::uint64_t raddr, std::uint32_t rkey,
                                std::uint32_t imm_be, bool signaled) = 0;
    virtual void post_recv(std::uint64_t wr_id, const Sge& sge) = 0;
    // Up to `max` completions of the QP's completion queue.
    virtual int poll(WorkCompletion* out, int max) = 0;
    virtual std::uint32_t max_inline() const = 0;
    virtual void fill_local_info(RdmaPeerInfo* info) const = 0;
    // INIT -> RTR -> RTS against the peer.
    virtual void connect(const RdmaPeerInfo& peer) = 0;
};

class VerbsDevice {
public:
    virtual ~VerbsDevice() = default;
    virtual std::string name() const = 0;
    virtual std::unique_ptr<MemoryRegion> register_host(void* addr, std::size_t bytes) = 0;
    // GPU memory: tries dma-buf first, then the peer-memory path; never falls back to host memory.
    virtual std::unique_ptr<MemoryRegion> register_device(void* addr, std::size_t bytes) = 0;
    virtual std::unique_ptr<QueuePair> create_qp(int send_depth, int recv_depth) = 0;
    virtual std::uint8_t active_mtu() const = 0;
};

// In-process loopback provider.  Two QPs created from the same device and connected to each other
// exchange data through plain memory copies.
std::shared_ptr<VerbsDevice> make_loopback_device(const std::string& name = "loopback0");

// libibverbs provider, or nullptr (with `why`) when libibverbs.so.1 cannot be loaded or no usable
// device exists.
std::shared_ptr<VerbsDevice> open_ibverbs_device(const RdmaConfig& config, std::string* why);

}  // namespace nano_nccl::rdma
