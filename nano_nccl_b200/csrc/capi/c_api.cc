// C ABI v2 over the C++ Communicator.
//
// Parity: reference src/c_api.cc:14-27, 98-158, 162-406 — thread-local 1 KiB diagnostic cleared
// by every stateful call, pure queries (abi_version / status_string / get_last_error) leave it
// alone, NULL destroy succeeds, NULL handle -> INVALID_ARGUMENT mentioning "communicator", the C
// layer pre-validates descriptors (null pointers, zero count, in-place, overlap, overflow,
// enum range) before reaching C++, C++ exceptions become status codes.
#include "capi/c_api_internal.h"

#include "core/error.h"
#include "nano_nccl/nano_nccl_ext.h"

#include <cstdint>
#include <cstdio>
#include <limits>
#include <vector>

namespace nano_nccl::c_api {

namespace {
thread_local char g_last_error[1024] = {0};
}

void begin_call() noexcept { g_last_error[0] = '\0'; }

nano_nccl_status_t fail(nano_nccl_status_t status, const char* message) noexcept {
    std::snprintf(g_last_error, sizeof(g_last_error), "%s", message != nullptr ? message : "");
    return status;
}

const char* last_error() noexcept { return g_last_error; }

nano_nccl_status_t require_handle(const nano_nccl_communicator_t* handle) noexcept {
    if (handle == nullptr || handle->communicator == nullptr) {
        return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "communicator must be non-null");
    }
    return NANO_NCCL_STATUS_SUCCESS;
}

bool to_dtype(nano_nccl_dtype_t v, DType* out) noexcept {
    if (v < NANO_NCCL_DTYPE_FLOAT || v > NANO_NCCL_DTYPE_BFLOAT16) return false;
    *out = static_cast<DType>(v);
    return true;
}
bool to_redop(nano_nccl_redop_t v, RedOp* out) noexcept {
    if (v < NANO_NCCL_REDOP_SUM || v > NANO_NCCL_REDOP_MIN) return false;
    *out = static_cast<RedOp>(v);
    return true;
}
bool to_transport(nano_nccl_transport_t v, TransportKind* out) noexcept {
    if (v < NANO_NCCL_TRANSPORT_AUTO || v > NANO_NCCL_TRANSPORT_RDMA) return false;  // mixed: result only
    *out = static_cast<TransportKind>(v);
    return true;
}
nano_nccl_transport_t from_transport(TransportKind v) noexcept {
    return static_cast<nano_nccl_transport_t>(static_cast<int>(v));
}

}  // namespace nano_nccl::c_api

namespace {

using namespace nano_nccl;
using namespace nano_nccl::c_api;

static_assert(static_cast<int>(DType::BFloat16) == NANO_NCCL_DTYPE_BFLOAT16, "enum order is ABI");
static_assert(static_cast<int>(RedOp::Min) == NANO_NCCL_REDOP_MIN, "enum order is ABI");
static_assert(static_cast<int>(TransportKind::Mixed) == NANO_NCCL_TRANSPORT_MIXED, "enum order is ABI");

// Descriptor checks shared by the three collectives.  send_factor / recv_factor scale `count` to
// the element counts of the two buffers (ReduceScatter input and AllGather output hold N chunks).
nano_nccl_status_t check_descriptor(const nano_nccl_communicator_t* handle, const void* send,
                                    void* recv, cudaStream_t stream, std::size_t count,
                                    nano_nccl_dtype_t dtype, bool send_scaled, bool recv_scaled) {
    // Communicators created for framework bindings accept the default stream and exact in-place
    // AllReduce; the C++ layer then applies its own (relaxed) checks.
    const bool relaxed = handle->communicator->relaxed_validation();
    if (send == nullptr || recv == nullptr || (stream == nullptr && !relaxed)) {
        return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "collective buffers and stream must be non-null");
    }
    if (count == 0) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "collective count must be positive");
    if (send == recv && relaxed && !send_scaled && !recv_scaled) return NANO_NCCL_STATUS_SUCCESS;
    if (send == recv) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "in-place collectives are unsupported");
    DType dt;
    if (!to_dtype(dtype, &dt)) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "unknown dtype");
    const std::size_t n = static_cast<std::size_t>(handle->communicator->global_rank_count());
    const std::size_t limit = std::numeric_limits<std::size_t>::max();
    const std::size_t esz = dtype_size(dt);
    if (count > limit / esz / n) {
        return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "collective byte count overflows size_t");
    }
    const std::size_t sb = count * esz * (send_scaled ? n : 1), rb = count * esz * (recv_scaled ? n : 1);
    const auto s0 = reinterpret_cast<std::uintptr_t>(send), r0 = reinterpret_cast<std::uintptr_t>(recv);
    if (s0 > limit - sb || r0 > limit - rb) {
        return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "collective buffer range overflows the address space");
    }
    if (s0 < r0 + rb && r0 < s0 + sb) {
        return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "send and receive buffers overlap; collectives are out-of-place");
    }
    return NANO_NCCL_STATUS_SUCCESS;
}

CommunicatorConfig from_ext(const nano_nccl_ext_config_t* c) {
    CommunicatorConfig cfg;
    if (c == nullptr) return cfg;
    cfg.device = c->device;
    NANO_REQUIRE_ARG(to_transport(c->transport, &cfg.transport), "unknown or unrequestable transport %d", c->transport);
    NANO_REQUIRE_ARG(c->algo >= 0 && c->algo <= 4, "unknown algorithm %d", c->algo);
    cfg.algo = static_cast<AlgoKind>(c->algo);
    cfg.enable_multicast = c->enable_multicast;
    cfg.wait_timeout_us = c->wait_timeout_us;
    cfg.relaxed_validation = c->relaxed_validation != 0;
    return cfg;
}

}  // namespace

extern "C" {

uint32_t nano_nccl_abi_version(void) { return NANO_NCCL_ABI_VERSION; }

const char* nano_nccl_status_string(nano_nccl_status_t status) {
    switch (status) {
        case NANO_NCCL_STATUS_SUCCESS: return "success";
        case NANO_NCCL_STATUS_INVALID_ARGUMENT: return "invalid argument";
        case NANO_NCCL_STATUS_UNSUPPORTED: return "unsupported";
        case NANO_NCCL_STATUS_ERROR: return "error";
        default: return "unknown status";
    }
}

const char* nano_nccl_get_last_error(void) { return nano_nccl::c_api::last_error(); }

nano_nccl_status_t nano_nccl_destroy_communicator(nano_nccl_communicator_t* communicator) {
    begin_call();
    if (communicator == nullptr) return NANO_NCCL_STATUS_SUCCESS;
    return guarded([&] { delete communicator; });
}

nano_nccl_status_t nano_nccl_all_reduce(nano_nccl_communicator_t* communicator,
                                        const nano_nccl_all_reduce_args_t* args) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (args == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "args must be non-null");
    if (auto s = check_descriptor(communicator, args->send_buffer, args->recv_buffer, args->stream,
                                  args->count, args->dtype, false, false)) return s;
    AllReduceArgs a;
    if (!to_dtype(args->dtype, &a.dtype)) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "unknown dtype");
    if (!to_redop(args->redop, &a.redop)) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "unknown reduction operator");
    a.send_buffer = args->send_buffer;
    a.recv_buffer = args->recv_buffer;
    a.stream = args->stream;
    a.count = args->count;
    return guarded([&] { communicator->communicator->all_reduce(a); });
}

nano_nccl_status_t nano_nccl_reduce_scatter(nano_nccl_communicator_t* communicator,
                                            const nano_nccl_reduce_scatter_args_t* args) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (args == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "args must be non-null");
    if (auto s = check_descriptor(communicator, args->send_buffer, args->recv_buffer, args->stream,
                                  args->recv_count, args->dtype, true, false)) return s;
    ReduceScatterArgs a;
    if (!to_dtype(args->dtype, &a.dtype)) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "unknown dtype");
    if (!to_redop(args->redop, &a.redop)) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "unknown reduction operator");
    a.send_buffer = args->send_buffer;
    a.recv_buffer = args->recv_buffer;
    a.stream = args->stream;
    a.recv_count = args->recv_count;
    return guarded([&] { communicator->communicator->reduce_scatter(a); });
}

nano_nccl_status_t nano_nccl_all_gather(nano_nccl_communicator_t* communicator,
                                        const nano_nccl_all_gather_args_t* args) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (args == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "args must be non-null");
    if (auto s = check_descriptor(communicator, args->send_buffer, args->recv_buffer, args->stream,
                                  args->send_count, args->dtype, false, true)) return s;
    AllGatherArgs a;
    if (!to_dtype(args->dtype, &a.dtype)) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "unknown dtype");
    a.send_buffer = args->send_buffer;
    a.recv_buffer = args->recv_buffer;
    a.stream = args->stream;
    a.send_count = args->send_count;
    return guarded([&] { communicator->communicator->all_gather(a); });
}

nano_nccl_status_t nano_nccl_check_async_error(const nano_nccl_communicator_t* communicator) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    return guarded([&] { communicator->communicator->check_async_error(); });
}

nano_nccl_status_t nano_nccl_local_rank_count(const nano_nccl_communicator_t* communicator, int* rank_count) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (rank_count == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "rank_count must be non-null");
    *rank_count = communicator->communicator->local_rank_count();
    return NANO_NCCL_STATUS_SUCCESS;
}

nano_nccl_status_t nano_nccl_global_rank_count(const nano_nccl_communicator_t* communicator, int* rank_count) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (rank_count == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "rank_count must be non-null");
    *rank_count = communicator->communicator->global_rank_count();
    return NANO_NCCL_STATUS_SUCCESS;
}

nano_nccl_status_t nano_nccl_transport(const nano_nccl_communicator_t* communicator,
                                       nano_nccl_transport_t* transport) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (transport == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "transport must be non-null");
    *transport = from_transport(communicator->communicator->transport());
    return NANO_NCCL_STATUS_SUCCESS;
}

nano_nccl_status_t nano_nccl_edge_transport(const nano_nccl_communicator_t* communicator,
                                            int source_global_rank, nano_nccl_transport_t* transport) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (transport == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "transport must be non-null");
    return guarded([&] { *transport = from_transport(communicator->communicator->edge_transport(source_global_rank)); });
}

nano_nccl_status_t nano_nccl_edge_uses_gdr(const nano_nccl_communicator_t* communicator,
                                           int source_global_rank, int* uses_gdr) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (uses_gdr == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "uses_gdr must be non-null");
    return guarded([&] { *uses_gdr = communicator->communicator->edge_uses_gdr(source_global_rank) ? 1 : 0; });
}

// ------------------------------------------------------------------------------------------------
// Extensions.

nano_nccl_status_t nano_nccl_create_tcp_communicator(const char* addr, int port, int rank, int size,
                                                     const nano_nccl_ext_config_t* config,
                                                     nano_nccl_communicator_t** communicator) {
    begin_call();
    if (communicator == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "communicator output must be non-null");
    *communicator = nullptr;
    return guarded([&] {
        std::shared_ptr<Bootstrap> bootstrap = make_tcp_bootstrap(addr != nullptr ? addr : "127.0.0.1", port, rank, size);
        auto handle = std::make_unique<NanoNcclCommunicator>();
        handle->communicator = create_communicator(bootstrap, from_ext(config));
        *communicator = handle.release();
    });
}

nano_nccl_status_t nano_nccl_create_callback_communicator(nano_nccl_allgather_fn allgather, void* user,
                                                          int rank, int size,
                                                          const nano_nccl_ext_config_t* config,
                                                          nano_nccl_communicator_t** communicator) {
    begin_call();
    if (communicator == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "communicator output must be non-null");
    *communicator = nullptr;
    if (allgather == nullptr && size > 1) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "allgather callback must be non-null");
    return guarded([&] {
        BootstrapCallbacks cb;
        cb.rank = rank;
        cb.size = size;
        cb.all_gather = [allgather, user](const void* in, void* out, std::size_t bytes) { allgather(user, in, out, bytes); };
        std::shared_ptr<Bootstrap> bootstrap = make_callback_bootstrap(std::move(cb));
        auto handle = std::make_unique<NanoNcclCommunicator>();
        handle->communicator = create_communicator(bootstrap, from_ext(config));
        *communicator = handle.release();
    });
}

int nano_nccl_bootstrap_selftest(nano_nccl_allgather_fn allgather, void* user, int rank, int size) {
    if (allgather == nullptr || size < 1 || rank < 0 || rank >= size) return 1;
    try {
        BootstrapCallbacks cb;
        cb.rank = rank;
        cb.size = size;
        cb.all_gather = [allgather, user](const void* in, void* out, std::size_t bytes) { allgather(user, in, out, bytes); };
        auto b = make_callback_bootstrap(std::move(cb));
        for (std::size_t words : {std::size_t{1}, std::size_t{17}, std::size_t{256}}) {
            std::vector<std::uint32_t> mine(words), all(words * static_cast<std::size_t>(size));
            for (std::size_t i = 0; i < words; ++i) mine[i] = static_cast<std::uint32_t>(rank * 1000003u + i);
            b->all_gather(mine.data(), all.data(), words * sizeof(std::uint32_t));
            for (int r = 0; r < size; ++r) {
                for (std::size_t i = 0; i < words; ++i) {
                    if (all[r * words + i] != static_cast<std::uint32_t>(r * 1000003u + i)) return 2;
                }
            }
        }
        b->barrier();
        if (b->all_reduce_min(rank) != 0 || b->all_reduce_max(rank) != size - 1) return 3;
        return 0;
    } catch (...) {
        return 4;
    }
}

nano_nccl_status_t nano_nccl_rank(const nano_nccl_communicator_t* communicator, int* rank) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (rank == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "rank must be non-null");
    *rank = communicator->communicator->rank();
    return NANO_NCCL_STATUS_SUCCESS;
}

nano_nccl_status_t nano_nccl_multicast_available(const nano_nccl_communicator_t* communicator, int* available) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (available == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "available must be non-null");
    *available = communicator->communicator->multicast_available() ? 1 : 0;
    return NANO_NCCL_STATUS_SUCCESS;
}

nano_nccl_status_t nano_nccl_set_algo(nano_nccl_communicator_t* communicator, nano_nccl_algo_t algo) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (algo < 0 || algo > 4) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "unknown algorithm");
    communicator->communicator->set_algo(static_cast<AlgoKind>(algo));
    return NANO_NCCL_STATUS_SUCCESS;
}

nano_nccl_status_t nano_nccl_set_grid_override(nano_nccl_communicator_t* communicator, int ctas) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (ctas < 0 || ctas > 160) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "grid override must be within 0..160");
    communicator->communicator->set_grid_override(ctas);
    return NANO_NCCL_STATUS_SUCCESS;
}

nano_nccl_status_t nano_nccl_last_algo(const nano_nccl_communicator_t* communicator, nano_nccl_algo_t* algo) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (algo == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "algo must be non-null");
    *algo = static_cast<nano_nccl_algo_t>(communicator->communicator->last_algo());
    return NANO_NCCL_STATUS_SUCCESS;
}

nano_nccl_status_t nano_nccl_symmetric_alloc(nano_nccl_communicator_t* communicator, size_t bytes, void** ptr) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (ptr == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "ptr must be non-null");
    return guarded([&] { *ptr = communicator->communicator->symmetric_alloc(bytes); });
}

nano_nccl_status_t nano_nccl_symmetric_free(nano_nccl_communicator_t* communicator, void* ptr) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    return guarded([&] { communicator->communicator->symmetric_free(ptr); });
}

nano_nccl_status_t nano_nccl_register_buffer(nano_nccl_communicator_t* communicator, void* ptr, size_t bytes) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    return guarded([&] { communicator->communicator->register_buffer(ptr, bytes); });
}

nano_nccl_status_t nano_nccl_deregister_buffer(nano_nccl_communicator_t* communicator, void* ptr) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    return guarded([&] { communicator->communicator->deregister_buffer(ptr); });
}

nano_nccl_status_t nano_nccl_peer_pointer(const nano_nccl_communicator_t* communicator, const void* ptr,
                                          int peer_rank, void** peer_ptr) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (peer_ptr == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "peer_ptr must be non-null");
    return guarded([&] { *peer_ptr = communicator->communicator->peer_pointer(ptr, peer_rank); });
}

nano_nccl_status_t nano_nccl_multicast_pointer(const nano_nccl_communicator_t* communicator, const void* ptr,
                                               void** mc_ptr) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (mc_ptr == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "mc_ptr must be non-null");
    return guarded([&] { *mc_ptr = communicator->communicator->multicast_pointer(ptr); });
}

nano_nccl_status_t nano_nccl_barrier(nano_nccl_communicator_t* communicator, cudaStream_t stream) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    return guarded([&] { communicator->communicator->barrier(stream); });
}

nano_nccl_status_t nano_nccl_get_stats(const nano_nccl_communicator_t* communicator, nano_nccl_stats_t* stats) {
    begin_call();
    if (auto s = require_handle(communicator)) return s;
    if (stats == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "stats must be non-null");
    const CommunicatorStats st = communicator->communicator->stats();
    *stats = nano_nccl_stats_t{st.launches, st.oneshot, st.twoshot, st.nvls, st.ring, st.zero_copy, st.local_only, st.pipelined};
    return NANO_NCCL_STATUS_SUCCESS;
}

}  // extern "C"
