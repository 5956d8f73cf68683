// Communicator runtime: bootstrap-time setup (topology, symmetric arena, multicast), argument
// validation, algorithm choice, kernel launch, cross-stream ordering, asynchronous error
// reporting and teardown.
//
// Parity: reference src/collective/all_reduce/communicator.cu:162-1503 (Communicator::Impl) and
// mpi_communicator.cc:297-410 (bootstrap sequence).  Kept: the validation rules and their order
// (check_async_error, then validate_args: count > 0, non-null buffers and stream, byte-count
// overflow, any overlap of the send and receive ranges rejected, unsupported redop rejected);
// collectives of one communicator are serialised even across different user streams; after a
// latched asynchronous error every call throws the same stable message; device selection is
// agreed collectively so that no rank is left waiting in a control collective.
#include "collective/communicator_impl.h"
#include "collective/teardown.h"
#include "collective/signature.h"

#include "core/env.h"
#include "transport/ring/ring_path.h"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <limits>

namespace nano_nccl {

namespace {

constexpr std::int64_t kDefaultTimeoutUs = 20'000'000;

bool ranges_overlap(const void* a, std::size_t a_bytes, const void* b, std::size_t b_bytes) {
    const auto a0 = reinterpret_cast<std::uintptr_t>(a), b0 = reinterpret_cast<std::uintptr_t>(b);
    return a0 < b0 + b_bytes && b0 < a0 + a_bytes;
}

bool checked_mul(std::size_t a, std::size_t b, std::size_t* out) {
    if (b != 0 && a > std::numeric_limits<std::size_t>::max() / b) return false;
    *out = a * b;
    return true;
}

const char* phase_name(std::uint32_t phase) {
    switch (phase) {
        case 1: return "after the push / copy-in phase";
        case 2: return "after the reduce / broadcast phase";
        case 9: return "in a barrier";
        default: return "in a fused GEMM wait";
    }
}

// Largest message of the flag-in-data kernels when the environment does not say: 1 MiB.  Measured (p50, device-timed,
// bf16): two ranks 12.3-12.8 us against 14.5-16.3 us at 256 KiB and level at 1 MiB; eight ranks (multimem pushes)
// geomean of NCCL time / this library's time over the 15 cells of the grid 1.37 with them against 1.25 without, no
// cell slower than NCCL.  Four ranks take the same code path as eight.
std::int64_t default_ll_max_bytes(int nranks) { return nranks >= 2 ? (1 << 20) : 0; }

}  // namespace

// ------------------------------------------------------------------------------------------------
Communicator::Impl::Impl(std::shared_ptr<Bootstrap> bootstrap, const CommunicatorConfig& config)
    : bootstrap_(std::move(bootstrap)), config_(config) {
    NANO_REQUIRE_ARG(bootstrap_ != nullptr, "a communicator needs a bootstrap");
    rank_ = bootstrap_->rank();
    nranks_ = bootstrap_->size();
    device_ = config.device;
    NANO_REQUIRE_ARG(nranks_ >= 1 && nranks_ <= kMaxRanks,
                     "communicator size %d must be within 1..%d", nranks_, kMaxRanks);

    // 1. device selection, agreed by all ranks (reference mpi_communicator.cc:44-89)
    bootstrap_->run_agreed("device selection", [&] {
        int count = 0;
        CUDA_CHECK_THROW(cudaGetDeviceCount(&count));
        NANO_REQUIRE_ARG(device_ >= 0 && device_ < count,
                         "config.device %d is not a visible CUDA device (%d visible)", device_, count);
        CUDA_CHECK_THROW(cudaSetDevice(device_));
        CUDA_CHECK_THROW(cudaFree(nullptr));
    });

    // 2. who is where (reference :91-141, 215-233)
    RankInfo mine = describe_local_rank(*bootstrap_, device_);
    mine.multicast = device_supports_multicast(device_) ? 1 : 0;
    ranks_.resize(static_cast<std::size_t>(nranks_));
    bootstrap_->all_gather(&mine, ranks_.data(), sizeof(RankInfo));
    bootstrap_->run_agreed("device uniqueness check", [&] { validate_unique_devices(ranks_); });

    // 3. peer-access probe towards the ring successor (reference mpi_p2p.cc:235-289 probes with a
    //    1-byte IPC handle; here the CUDA P2P attribute answers the same question)
    {
        const RankInfo& next = ranks_[(rank_ + 1) % nranks_];
        int can = nranks_ == 1 ? 1 : 0;
        if (nranks_ > 1 && next.node_id == mine.node_id) {
            // The successor's ordinal is only meaningful in this process's numbering when both see
            // the same devices; match it by UUID instead.
            int count = 0;
            cudaGetDeviceCount(&count);
            for (int d = 0; d < count; ++d) {
                cudaDeviceProp prop{};
                if (cudaGetDeviceProperties(&prop, d) != cudaSuccess) continue;
                if (std::memcmp(prop.uuid.bytes, next.uuid.data(), 16) == 0) {
                    int access = 0;
                    if (cudaDeviceCanAccessPeer(&access, device_, d) == cudaSuccess) can = access;
                    break;
                }
            }
            cudaGetLastError();
            // A peer hidden by CUDA_VISIBLE_DEVICES cannot be probed by ordinal; NVSwitch systems
            // are fully connected, so fall back to "same host and multicast-capable => reachable".
            if (can == 0 && mine.multicast != 0 && next.multicast != 0) can = 1;
        }
        mine.can_access_next = can;
        bootstrap_->all_gather(&mine, ranks_.data(), sizeof(RankInfo));
    }

    // 4. transports per ring edge (reference mpi_communicator.cc:235-293)
    bootstrap_->run_agreed("transport resolution", [&] {
        topology_.global_rank_count = nranks_;
        topology_.local_rank_offset = rank_;
        topology_.devices = {device_};
        topology_.distributed = true;
        topology_.edge_kinds = resolve_edge_transports(config_.transport, ranks_);
        validate_topology(topology_);
    });
    plan_.edge_kinds = topology_.edge_kinds;

    // 5. configuration
    timeout_us_ = config_.wait_timeout_us > 0
                      ? config_.wait_timeout_us
                      : env::integer("NANO_NCCL_WAIT_TIMEOUT_US", kDefaultTimeoutUs, 1000, 3'600'000'000ll);
    bool want_mc = config_.enable_multicast < 0 ? env::flag("NANO_NCCL_NVLS", true)
                                                : config_.enable_multicast != 0;
    relaxed_validation_ = env::flag("NANO_NCCL_RELAXED_VALIDATION", false);
    // Shifting odd CTAs by half a tile was meant to overlap the egress-heavy push phase of some
    // CTAs with the ingress-heavy broadcast phase of others.  Measured, the smaller tiles and extra
    // barriers cost more than the overlap gains (64 MiB two-shot AllReduce: 4 GPUs 248 us skewed
    // vs 202 us plain; 2 GPUs 208 vs 174), so it is off unless asked for.
    skew_ = env::flag("NANO_NCCL_SKEW", false) && nranks_ > 2;
    debug_signatures_ = env::flag("NANO_NCCL_DEBUG_SIGNATURES", false);
    if (auto level = env::get("NANO_NCCL_DEBUG")) {
        NANO_REQUIRE_ARG(level->empty() || *level == "0" || *level == "info" || *level == "trace",
                         "NANO_NCCL_DEBUG must be unset, 0, info or trace, got '%s'", level->c_str());
        debug_level_ = *level == "info" ? 1 : *level == "trace" ? 2 : 0;
    }
    push_tma_ = env::flag("NANO_NCCL_PUSH_TMA", false);
    // Messages of at least this many bytes (AllReduce message; ReduceScatter / AllGather: the whole N-chunk buffer)
    // take the software-pipelined kernels; 0 (the default) switches them off.  Off because they measured slower than
    // the plain kernels on two B200 at every depth and tile size tried (64 MiB AllReduce 248 us against 176 us,
    // 16 MiB ReduceScatter 60 us against 39 us): every signal costs a release fence of about 5 us on a busy link,
    // and one signalling warp issues two of them per iteration whatever the tile size.
    pipe_min_bytes_ = static_cast<std::size_t>(env::integer("NANO_NCCL_PIPE_MIN_BYTES", 0, 0, 1ll << 40));
    pipe_tile_bytes_ = static_cast<std::size_t>(env::integer("NANO_NCCL_PIPE_TILE_BYTES", 0, 0, 1 << 20));
    pipe_depth_ = static_cast<int>(env::integer("NANO_NCCL_PIPE_DEPTH", 0, 0, dev::kMaxPipeDepth));
    if (auto algo = env::get("NANO_NCCL_PIPE_ALGO")) {
        NANO_REQUIRE_ARG(parse_algo(algo->c_str(), &pipe_algo_) && (pipe_algo_ == AlgoKind::Auto || pipe_algo_ == AlgoKind::TwoShot || pipe_algo_ == AlgoKind::Nvls),
                         "NANO_NCCL_PIPE_ALGO must be auto, twoshot or nvls, got '%s'", algo->c_str());
    }
    tile_cap_ = static_cast<std::size_t>(env::integer("NANO_NCCL_TILE_BYTES", 0, 0, 1 << 20));

    // 6. NVLink data plane: symmetric arena + signal pads when every edge is GPU peer-to-peer
    status_ = MappedU32Array(8, gpu_numa_node(device_));
    abort_ = MappedU32Array(8, gpu_numa_node(device_));
    nvlink_path_ = plan_.all_p2p() || nranks_ == 1;
    if (nvlink_path_) {
        if (nranks_ > 1) fds_ = std::make_unique<FdChannel>(*bootstrap_);
        SymmetricMemory::Options options;
        options.want_multicast = want_mc && nranks_ > 1;
        options.zero = true;
        arena_ = SymmetricMemory::create(*bootstrap_, fds_.get(), device_, dev::kArenaBytes, options);
        state_ = RawDeviceBuffer(device_, sizeof(dev::BlockState) * dev::kMaxBlocks, true);
        fill_device_context();
        // Flag-in-data kernels for small messages, in a staging segment of their own.  NANO_NCCL_LL_MAX_BYTES is the
        // largest message that takes them (AllReduce message; ReduceScatter / AllGather: the whole N-chunk buffer),
        // 0 switches them off.  Default: kDefaultLLMaxBytes where they were measured faster than the barrier
        // kernels (see default_ll_max_bytes).
        ll_max_bytes_ = static_cast<std::size_t>(env::integer("NANO_NCCL_LL_MAX_BYTES", default_ll_max_bytes(nranks_), 0, 16 << 20));
        if (nranks_ > 1) {
            NANO_REQUIRE_ARG(bootstrap_->all_reduce_min(static_cast<std::int64_t>(ll_max_bytes_)) ==
                                 bootstrap_->all_reduce_max(static_cast<std::int64_t>(ll_max_bytes_)),
                             "ranks disagree on NANO_NCCL_LL_MAX_BYTES");
            if (ll_max_bytes_ != 0) {
                ll_arena_ = SymmetricMemory::create(*bootstrap_, fds_.get(), device_, dev::kLLArenaBytes, options);
                for (int r = 0; r < nranks_; ++r) ll_dev_.stage[r] = static_cast<char*>(ll_arena_->peer(r));
                ll_dev_.stage_mc = static_cast<char*>(ll_arena_->multicast());
            }
        }
    }
    tuner_ = std::make_unique<Tuner>(nranks_, multicast_available());
    if (config_.algo != AlgoKind::Auto) tuner_->set_forced_algo(config_.algo);
    completion_ = Event::create(false);
    // 7. Ring / Simple fallback data plane: always when some edge is not GPU peer-to-peer, on
    //    request otherwise (algo = ring, or NANO_NCCL_RING=1).  Every rank must decide alike.
    const bool want_ring = nranks_ > 1 && (!nvlink_path_ || tuner_->forced_algo() == AlgoKind::Ring ||
                                           env::flag("NANO_NCCL_RING", false));
    NANO_REQUIRE_ARG(bootstrap_->all_reduce_min(want_ring ? 1 : 0) == bootstrap_->all_reduce_max(want_ring ? 1 : 0),
                     "ranks disagree on whether the Ring/Simple path is enabled");
    if (want_ring) ring_ = create_ring_path(*this);
    CUDA_CHECK_THROW(cudaDeviceSynchronize());
    bootstrap_->barrier();
    if (debug_level_ >= 1) {
        std::fprintf(stderr,
                     "nano_nccl: rank %d of %d on device %d: transport %s, NVLink path %s, multicast %s%s%s, ring %s, "
                     "wait limit %lld us, LL up to %zu bytes\n",
                     rank_, nranks_, device_, transport_name(plan_.resolved_kind()), nvlink_path_ ? "on" : "off",
                     multicast_available() ? "on" : "off",
                     (arena_ != nullptr && !multicast_available() && !arena_->multicast_note().empty()) ? " (" : "",
                     (arena_ != nullptr && !multicast_available() && !arena_->multicast_note().empty())
                         ? (arena_->multicast_note() + ")").c_str() : "",
                     ring_ != nullptr ? "ready" : "not created", static_cast<long long>(timeout_us_), ll_max_bytes_);
    }
}

void Communicator::Impl::fill_device_context() {
    dev_ = dev::CommDev{};
    dev_.rank = rank_;
    dev_.nranks = nranks_;
    for (int r = 0; r < nranks_; ++r) {
        char* base = static_cast<char*>(arena_->peer(r));
        dev_.pad[r] = reinterpret_cast<std::uint32_t*>(base);
        dev_.stage[r] = base + dev::kPadBytes;
    }
    dev_.stage_mc = arena_->multicast() != nullptr
                        ? static_cast<char*>(arena_->multicast()) + dev::kPadBytes
                        : nullptr;
    dev_.state = static_cast<dev::BlockState*>(state_.data());
    dev_.status = status_.device();
    dev_.abort_flag = abort_.device();
    dev_.timeout_ns = static_cast<unsigned long long>(timeout_us_) * 1000ull;
}

Communicator::Impl::~Impl() {
    // Teardown order (reference communicator.cu:194-228): stop waiting kernels if an error is
    // latched, drain this rank's own work, then release transports.  Peers are not consulted: a
    // rank may leave while others are still alive (asymmetric teardown is legal).
    if (status_.size() != 0 && status_.host()[0] != 0 && abort_.size() != 0) {
        abort_.host()[0] = 1;
    }
    cudaError_t drained = cudaSetDevice(device_);
    if (drained == cudaSuccess) drained = cudaDeviceSynchronize();
    cudaGetLastError();
    if (env::flag("NANO_NCCL_TEST_TEARDOWN_FAILURE", false)) drained = cudaErrorUnknown;  // host-side injection for tests
    TeardownAction action = TeardownAction::Quarantine;
    try {
        action = decide_teardown(drained != cudaSuccess, env::get("NANO_NCCL_TEARDOWN").value_or(""));
    } catch (const std::exception& e) {
        std::fprintf(stderr, "nano_nccl: %s; using 'quarantine'\n", e.what());
        action = drained != cudaSuccess ? TeardownAction::Quarantine : TeardownAction::Release;
    }
    if (action != TeardownAction::Release) {
        std::fprintf(stderr,
                     "nano_nccl: rank %d could not drain its GPU work while destroying a communicator (%s); %s\n", rank_,
                     cudaGetErrorString(drained),
                     action == TeardownAction::Abort
                         ? "NANO_NCCL_TEARDOWN=abort: ending the process"
                         : "leaving its device memory mapped (a kernel or a peer may still use it)");
        if (action == TeardownAction::Abort) std::terminate();
        // Quarantine: the owners are released without running their destructors.
        (void)ring_.release();
        for (auto& segment : heap_) (void)segment.release();
        (void)ll_arena_.release();
        (void)arena_.release();
        (void)fds_.release();
        state_.leak();
        barrier_words_.leak();
        return;
    }
    ring_.reset();
    heap_.clear();
    ll_arena_.reset();
    arena_.reset();
}

// ------------------------------------------------------------------------------------------------
void Communicator::Impl::check_async_error() const {
    if (!async_error_.empty()) throw std::runtime_error(async_error_);
    if (status_.size() != 0) {
        const volatile std::uint32_t* s = status_.host();
        const std::uint32_t code = s[0];
        if (code != 0) {
            const char* what = code == dev::kStatusWaitTimeout ? "a bounded device wait ran out"
                               : code == dev::kStatusAborted   ? "a device wait was aborted by the host"
                                                               : "a device-side check failed";
            async_error_ = format_message(
                "asynchronous communicator error on rank %d: %s while waiting for rank %u %s (block %u); "
                "the communicator is unusable",
                rank_, what, s[1], phase_name(s[2]), s[3]);
            throw std::runtime_error(async_error_);
        }
    }
    if (ring_ != nullptr) {
        std::string message;
        if (ring_->async_error(&message)) {
            async_error_ = message;
            throw std::runtime_error(async_error_);
        }
    }
}

void Communicator::Impl::validate_args(const void* send, void* recv, cudaStream_t stream,
                                       std::size_t count, std::size_t send_elems,
                                       std::size_t recv_elems, DType dtype, int redop,
                                       bool allow_exact_in_place) const {
    NANO_REQUIRE_ARG(count > 0, "collective count must be positive");
    NANO_REQUIRE_ARG(send != nullptr && recv != nullptr, "collective buffers must be non-null");
    if (!relaxed_validation_ && !config_relaxed()) {
        NANO_REQUIRE_ARG(stream != nullptr, "collective stream must be non-null");
    }
    NANO_REQUIRE_ARG(static_cast<int>(dtype) >= 0 && static_cast<int>(dtype) <= 2, "unsupported dtype");
    NANO_REQUIRE_ARG(redop >= 0 && redop <= 3, "unsupported reduction operator");
    std::size_t send_bytes = 0, recv_bytes = 0;
    NANO_REQUIRE_ARG(checked_mul(send_elems, dtype_size(dtype), &send_bytes) &&
                         checked_mul(recv_elems, dtype_size(dtype), &recv_bytes),
                     "collective byte count overflows size_t");
    if (send == recv && allow_exact_in_place && (relaxed_validation_ || config_relaxed())) return;
    NANO_REQUIRE_ARG(send != recv, "in-place collectives are unsupported");
    NANO_REQUIRE_ARG(!ranges_overlap(send, send_bytes, recv, recv_bytes),
                     "send and receive buffers overlap; collectives are out-of-place");
}

void Communicator::Impl::order_after_previous(cudaStream_t stream) {
    // Collectives of one communicator share staging and signal pads, so they are serialised even
    // when the caller uses different streams (reference communicator.cu:1034-1045).  The event is
    // only needed when the stream changes: same-stream launches are ordered already.
    if (has_last_stream_ && stream != last_stream_) {
        completion_.record(last_stream_);
        CUDA_CHECK_THROW(cudaStreamWaitEvent(stream, completion_.get(), 0));
    }
    last_stream_ = stream;
    has_last_stream_ = true;
}

void Communicator::Impl::check_signature(CollectiveKind kind, std::size_t count, DType dtype, int redop, bool in_place) {
    const std::uint64_t sequence = call_sequence_++;
    if (!debug_signatures_ || nranks_ == 1) return;
    CallSignature mine;
    mine.collective = static_cast<std::uint32_t>(kind);
    mine.dtype = static_cast<std::uint32_t>(dtype);
    mine.redop = static_cast<std::uint32_t>(redop);
    mine.in_place = in_place ? 1u : 0u;
    mine.count = count;
    mine.sequence = sequence;
    const std::string difference = compare_signatures(*bootstrap_, mine);
    if (!difference.empty()) throw std::invalid_argument(difference);
}

void Communicator::Impl::local_copy(const void* send, void* recv, std::size_t bytes,
                                    cudaStream_t stream) {
    CUDA_CHECK_THROW(cudaMemcpyAsync(recv, send, bytes, cudaMemcpyDeviceToDevice, stream));
    ++stats_.local_only;
}

SymmetricMemory* Communicator::Impl::find_symmetric(const void* ptr, std::size_t bytes) const noexcept {
    for (const auto& seg : heap_) {
        if (seg->contains(ptr, bytes)) return seg.get();
    }
    return nullptr;
}

void Communicator::Impl::all_reduce(const AllReduceArgs& a) {
    check_async_error();
    validate_args(a.send_buffer, a.recv_buffer, a.stream, a.count, a.count, a.count, a.dtype,
                  static_cast<int>(a.redop), /*allow_exact_in_place=*/true);
    check_signature(CollectiveKind::AllReduce, a.count, a.dtype, static_cast<int>(a.redop), a.send_buffer == a.recv_buffer);
    CUDA_CHECK_THROW(cudaSetDevice(device_));
    const std::size_t bytes = a.count * dtype_size(a.dtype);
    ++stats_.launches;
    if (nranks_ == 1) {
        // One rank: every operator is the identity (avg divides by 1).
        if (a.send_buffer != a.recv_buffer) local_copy(a.send_buffer, a.recv_buffer, bytes, a.stream);
        last_algo_ = AlgoKind::OneShot;
        return;
    }
    TunerDecision d = tuner_->decide(CollectiveKind::AllReduce, bytes, a.redop);
    if (!nvlink_path_) d.algo = AlgoKind::Ring;
    if (d.algo == AlgoKind::Ring) {
        run_ring(CollectiveKind::AllReduce, a.send_buffer, a.recv_buffer, a.count, a.dtype, a.redop, a.stream);
        return;
    }
    order_after_previous(a.stream);
    cudaError_t err = cudaSuccess;
    // Zero-copy: both buffers live in symmetric memory (possibly different segments), 16-byte
    // aligned, whole vectors.
    SymmetricMemory* seg = find_symmetric(a.send_buffer, bytes);
    SymmetricMemory* rseg = find_symmetric(a.recv_buffer, bytes);
    const bool zero_copy = seg != nullptr && rseg != nullptr && bytes % 16 == 0 &&
                           reinterpret_cast<std::uintptr_t>(a.send_buffer) % 16 == 0 &&
                           reinterpret_cast<std::uintptr_t>(a.recv_buffer) % 16 == 0;
    if (zero_copy) {
        const std::size_t so = static_cast<const char*>(a.send_buffer) - static_cast<const char*>(seg->local());
        const std::size_t ro = static_cast<const char*>(a.recv_buffer) - static_cast<const char*>(rseg->local());
        const bool adds = a.redop == RedOp::Sum || a.redop == RedOp::Avg;
        // In-place one-shot would let a fast rank overwrite data a slow rank still reads.
        AlgoKind algo = d.algo;
        if (algo == AlgoKind::OneShot && a.send_buffer == a.recv_buffer) algo = AlgoKind::TwoShot;
        if (algo == AlgoKind::Nvls && !(seg->multicast() != nullptr && rseg->multicast() != nullptr && adds)) {
            algo = AlgoKind::TwoShot;
        }
        const std::size_t per_rank = std::max<std::size_t>(bytes / nranks_, 1);
        const std::size_t per_cta = algo == AlgoKind::OneShot ? 8 * 1024 : 16 * 1024;
        const std::size_t work = algo == AlgoKind::OneShot ? bytes : per_rank;
        const int grid = std::max(1, std::min<int>(d.max_grid, static_cast<int>(work / per_cta) + 1));
        if (algo == AlgoKind::Nvls) {
            err = dev::launch_ar_nvls_symm(dev_, static_cast<char*>(seg->multicast()) + so,
                                           static_cast<char*>(rseg->multicast()) + ro, bytes, a.dtype, a.redop, grid,
                                           a.stream);
            ++stats_.nvls;
        } else {
            const void* src_peers[kMaxRanks];
            void* dst_peers[kMaxRanks];
            for (int r = 0; r < nranks_; ++r) {
                src_peers[r] = static_cast<const char*>(seg->peer(r)) + so;
                dst_peers[r] = static_cast<char*>(rseg->peer(r)) + ro;
            }
            err = dev::launch_ar_symm_p2p(dev_, src_peers, dst_peers, bytes, a.dtype, a.redop,
                                          algo == AlgoKind::OneShot, grid, a.stream);
            if (algo == AlgoKind::OneShot) ++stats_.oneshot; else ++stats_.twoshot;
        }
        ++stats_.zero_copy;
        last_algo_ = algo;
        CUDA_CHECK_THROW(err);
        return;
    }
    const bool adds = a.redop == RedOp::Sum || a.redop == RedOp::Avg;
    if (pipe_min_bytes_ != 0 && bytes >= pipe_min_bytes_ && d.algo != AlgoKind::OneShot) {
        // Large message: the software-pipelined kernels.  Through the switch when it can add (both link directions
        // carry about one message each); otherwise, and on two ranks, the two-shot form over peer stores.
        const bool through_switch = multicast_available() && adds &&
                                    (pipe_algo_ == AlgoKind::Nvls || (pipe_algo_ == AlgoKind::Auto && (nranks_ > 2 || d.algo == AlgoKind::Nvls)));
        if (through_switch) {
            const dev::Geometry g = dev::make_pipe_geometry(dev::Family::ArNvls, a.count, dtype_size(a.dtype), nranks_, d.max_grid, pipe_tile_bytes_, pipe_depth_);
            err = dev::launch_ar_nvls_pipe(dev_, a.send_buffer, a.recv_buffer, a.count, a.dtype, a.redop, g, a.stream);
            ++stats_.nvls;
            last_algo_ = AlgoKind::Nvls;
        } else {
            const dev::Geometry g = dev::make_pipe_geometry(dev::Family::ArTwoShot, a.count, dtype_size(a.dtype), nranks_, d.max_grid, pipe_tile_bytes_, pipe_depth_);
            err = dev::launch_ar_twoshot_pipe(dev_, a.send_buffer, a.recv_buffer, a.count, a.dtype, a.redop, push_multicast(), g, a.stream);
            ++stats_.twoshot;
            last_algo_ = AlgoKind::TwoShot;
        }
        ++stats_.pipelined;
        CUDA_CHECK_THROW(err);
        return;
    }
    if (d.algo == AlgoKind::Nvls) {
        const dev::Geometry g = dev::make_geometry(dev::Family::ArNvls, a.count, dtype_size(a.dtype), nranks_, d.max_grid, skew_, tile_cap_);
        err = dev::launch_ar_nvls(dev_, a.send_buffer, a.recv_buffer, a.count, a.dtype, a.redop, g, a.stream);
        ++stats_.nvls;
    } else if (d.algo == AlgoKind::OneShot && ll_arena_ != nullptr && bytes * static_cast<std::size_t>(nranks_) <= 2 * ll_max_bytes_) {
        // AllReduce: every rank receives N - 1 flagged copies (twice the bytes each), so the limit shrinks with the rank
        // count: ll_max_bytes on two ranks, a quarter of it on eight (measured there: 256 KiB 20.5 us against 24.7 us
        // for the barrier kernel, but 1 MiB 37.9 us against 30.7 us).
        const dev::Geometry g = dev::make_geometry(dev::Family::ArOneShot, a.count, dtype_size(a.dtype), nranks_, d.max_grid, false,
                                                   dev::ll_tile_cap_bytes(nranks_));
        err = dev::launch_ar_oneshot_ll(dev_, ll_dev_, a.send_buffer, a.recv_buffer, a.count, a.dtype, a.redop,
                                        push_multicast() && ll_dev_.stage_mc != nullptr, g, a.stream);
        ++stats_.oneshot;
    } else if (d.algo == AlgoKind::OneShot) {
        const dev::Geometry g = dev::make_geometry(dev::Family::ArOneShot, a.count, dtype_size(a.dtype), nranks_, d.max_grid, false, tile_cap_);
        err = dev::launch_ar_oneshot(dev_, a.send_buffer, a.recv_buffer, a.count, a.dtype, a.redop,
                                     push_multicast(), g, a.stream);
        ++stats_.oneshot;
    } else {
        const dev::Geometry g = dev::make_geometry(dev::Family::ArTwoShot, a.count, dtype_size(a.dtype), nranks_, d.max_grid, skew_, tile_cap_);
        err = dev::launch_ar_twoshot(dev_, a.send_buffer, a.recv_buffer, a.count, a.dtype, a.redop,
                                     push_multicast(), g, a.stream);
        ++stats_.twoshot;
    }
    last_algo_ = d.algo;
    CUDA_CHECK_THROW(err);
}

void Communicator::Impl::reduce_scatter(const ReduceScatterArgs& a) {
    check_async_error();
    std::size_t total = 0;
    NANO_REQUIRE_ARG(checked_mul(a.recv_count, static_cast<std::size_t>(nranks_), &total),
                     "collective element count overflows size_t");
    validate_args(a.send_buffer, a.recv_buffer, a.stream, a.recv_count, total, a.recv_count, a.dtype,
                  static_cast<int>(a.redop), false);
    check_signature(CollectiveKind::ReduceScatter, a.recv_count, a.dtype, static_cast<int>(a.redop), false);
    CUDA_CHECK_THROW(cudaSetDevice(device_));
    const std::size_t bytes = a.recv_count * dtype_size(a.dtype);
    ++stats_.launches;
    if (nranks_ == 1) {
        local_copy(a.send_buffer, a.recv_buffer, bytes, a.stream);
        last_algo_ = AlgoKind::OneShot;
        return;
    }
    TunerDecision d = tuner_->decide(CollectiveKind::ReduceScatter, bytes, a.redop);
    if (!nvlink_path_) d.algo = AlgoKind::Ring;
    if (d.algo == AlgoKind::Ring) {
        run_ring(CollectiveKind::ReduceScatter, a.send_buffer, a.recv_buffer, a.recv_count, a.dtype, a.redop, a.stream);
        return;
    }
    order_after_previous(a.stream);
    if (d.algo == AlgoKind::Nvls) {
        // Zero-copy through the switch: the input lives in multicast-bound symmetric memory, so rank r
        // reads the sum of chunk r with multimem.ld_reduce.  Anything that does not qualify uses the push kernel.
        const std::size_t total_bytes = total * dtype_size(a.dtype);
        SymmetricMemory* seg = find_symmetric(a.send_buffer, total_bytes);
        const bool adds = a.redop == RedOp::Sum || a.redop == RedOp::Avg;
        if (seg != nullptr && seg->multicast() != nullptr && adds && bytes % 16 == 0 &&
            reinterpret_cast<std::uintptr_t>(a.send_buffer) % 16 == 0 &&
            reinterpret_cast<std::uintptr_t>(a.recv_buffer) % 16 == 0) {
            const std::size_t so = static_cast<const char*>(a.send_buffer) - static_cast<const char*>(seg->local());
            const int grid = std::max(1, std::min<int>(d.max_grid, static_cast<int>(bytes / (16 * 1024)) + 1));
            const cudaError_t e = dev::launch_rs_nvls_symm(dev_, static_cast<const char*>(seg->multicast()) + so,
                                                           a.recv_buffer, bytes, a.dtype, a.redop, grid, a.stream);
            ++stats_.nvls;
            ++stats_.zero_copy;
            last_algo_ = AlgoKind::Nvls;
            CUDA_CHECK_THROW(e);
            return;
        }
    }
    if (ll_arena_ != nullptr && bytes * nranks_ <= ll_max_bytes_) {
        const dev::Geometry g = dev::make_geometry(dev::Family::ReduceScatter, a.recv_count, dtype_size(a.dtype), nranks_, d.max_grid,
                                                   false, dev::ll_tile_cap_bytes(nranks_));
        const cudaError_t e = dev::launch_rs_ll(dev_, ll_dev_, a.send_buffer, a.recv_buffer, a.recv_count, a.dtype, a.redop, g, a.stream);
        ++stats_.oneshot;
        last_algo_ = AlgoKind::OneShot;
        CUDA_CHECK_THROW(e);
        return;
    }
    if (pipe_min_bytes_ != 0 && bytes * nranks_ >= pipe_min_bytes_) {
        const dev::Geometry g = dev::make_pipe_geometry(dev::Family::ReduceScatter, a.recv_count, dtype_size(a.dtype), nranks_, d.max_grid, pipe_tile_bytes_, pipe_depth_);
        const cudaError_t e = dev::launch_rs_pipe(dev_, a.send_buffer, a.recv_buffer, a.recv_count, a.dtype, a.redop, g, a.stream);
        ++stats_.oneshot;
        ++stats_.pipelined;
        last_algo_ = AlgoKind::OneShot;
        CUDA_CHECK_THROW(e);
        return;
    }
    const dev::Geometry g = dev::make_geometry(dev::Family::ReduceScatter, a.recv_count, dtype_size(a.dtype), nranks_, d.max_grid, false, tile_cap_);
    const cudaError_t err = dev::launch_rs_push(dev_, a.send_buffer, a.recv_buffer, a.recv_count, a.dtype, a.redop, g, a.stream);
    ++stats_.oneshot;
    last_algo_ = AlgoKind::OneShot;
    CUDA_CHECK_THROW(err);
}

void Communicator::Impl::all_gather(const AllGatherArgs& a) {
    check_async_error();
    std::size_t total = 0;
    NANO_REQUIRE_ARG(checked_mul(a.send_count, static_cast<std::size_t>(nranks_), &total),
                     "collective element count overflows size_t");
    validate_args(a.send_buffer, a.recv_buffer, a.stream, a.send_count, a.send_count, total, a.dtype, 0, false);
    check_signature(CollectiveKind::AllGather, a.send_count, a.dtype, 0, false);
    CUDA_CHECK_THROW(cudaSetDevice(device_));
    const std::size_t bytes = a.send_count * dtype_size(a.dtype);
    ++stats_.launches;
    if (nranks_ == 1) {
        local_copy(a.send_buffer, a.recv_buffer, bytes, a.stream);
        last_algo_ = AlgoKind::OneShot;
        return;
    }
    TunerDecision d = tuner_->decide(CollectiveKind::AllGather, bytes, RedOp::Sum);
    if (!nvlink_path_) d.algo = AlgoKind::Ring;
    if (d.algo == AlgoKind::Ring) {
        run_ring(CollectiveKind::AllGather, a.send_buffer, a.recv_buffer, a.send_count, a.dtype, RedOp::Sum, a.stream);
        return;
    }
    order_after_previous(a.stream);
    if (d.algo == AlgoKind::Nvls) {
        // Zero-copy: the output lives in symmetric memory, so every rank stores its chunk straight into
        // slot `rank` of every rank's output (through the switch's multicast when there is more than one peer).
        const std::size_t total_bytes = total * dtype_size(a.dtype);
        SymmetricMemory* seg = find_symmetric(a.recv_buffer, total_bytes);
        if (seg != nullptr && bytes % 16 == 0 && reinterpret_cast<std::uintptr_t>(a.send_buffer) % 16 == 0 &&
            reinterpret_cast<std::uintptr_t>(a.recv_buffer) % 16 == 0) {
            const std::size_t ro = static_cast<char*>(a.recv_buffer) - static_cast<char*>(seg->local());
            void* peers[kMaxRanks] = {};
            for (int r = 0; r < nranks_; ++r) peers[r] = static_cast<char*>(seg->peer(r)) + ro;
            void* mc = (push_multicast() && seg->multicast() != nullptr) ? static_cast<char*>(seg->multicast()) + ro : nullptr;
            const int grid = std::max(1, std::min<int>(d.max_grid, static_cast<int>(bytes / (16 * 1024)) + 1));
            const cudaError_t e = dev::launch_ag_symm(dev_, a.send_buffer, peers, mc, bytes, grid, a.stream);
            ++stats_.zero_copy;
            last_algo_ = AlgoKind::Nvls;
            CUDA_CHECK_THROW(e);
            return;
        }
    }
    if (ll_arena_ != nullptr && bytes * nranks_ <= ll_max_bytes_) {
        const dev::Geometry g = dev::make_geometry(dev::Family::AllGather, a.send_count, dtype_size(a.dtype), nranks_, d.max_grid,
                                                   false, dev::ll_tile_cap_bytes(nranks_));
        const cudaError_t e = dev::launch_ag_ll(dev_, ll_dev_, a.send_buffer, a.recv_buffer, a.send_count, a.dtype,
                                                push_multicast() && ll_dev_.stage_mc != nullptr, g, a.stream);
        ++stats_.oneshot;
        last_algo_ = AlgoKind::OneShot;
        CUDA_CHECK_THROW(e);
        return;
    }
    if (pipe_min_bytes_ != 0 && bytes * nranks_ >= pipe_min_bytes_ && !push_tma_) {
        const dev::Geometry g = dev::make_pipe_geometry(dev::Family::AllGather, a.send_count, dtype_size(a.dtype), nranks_, d.max_grid, pipe_tile_bytes_, pipe_depth_);
        const cudaError_t e = dev::launch_ag_pipe(dev_, a.send_buffer, a.recv_buffer, a.send_count, a.dtype, push_multicast(), g, a.stream);
        ++stats_.oneshot;
        ++stats_.pipelined;
        last_algo_ = AlgoKind::OneShot;
        CUDA_CHECK_THROW(e);
        return;
    }
    const dev::Geometry g = dev::make_geometry(dev::Family::AllGather, a.send_count, dtype_size(a.dtype), nranks_, d.max_grid, false, tile_cap_);
    cudaError_t err = cudaErrorInvalidValue;
    if (push_tma_) err = dev::launch_ag_push_tma(dev_, a.send_buffer, a.recv_buffer, a.send_count, a.dtype, g, a.stream);
    if (err == cudaErrorInvalidValue) {
        err = dev::launch_ag_push(dev_, a.send_buffer, a.recv_buffer, a.send_count, a.dtype, push_multicast(), g, a.stream);
    }
    ++stats_.oneshot;
    last_algo_ = AlgoKind::OneShot;
    CUDA_CHECK_THROW(err);
}

void Communicator::Impl::run_ring(CollectiveKind kind, const void* send, void* recv, std::size_t count,
                                  DType dtype, RedOp op, cudaStream_t stream) {
    if (ring_ == nullptr) {
        throw std::runtime_error(
            "the Ring/Simple path is not available on this communicator (it is created on demand by "
            "ensure_ring(), a collective call)");
    }
    order_after_previous(stream);
    ring_->run(kind, send, recv, count, dtype, op, stream);
    ++stats_.ring;
    last_algo_ = AlgoKind::Ring;
}

void Communicator::Impl::barrier(cudaStream_t stream) {
    check_async_error();
    if (nranks_ == 1) return;
    CUDA_CHECK_THROW(cudaSetDevice(device_));
    if (!nvlink_path_) {
        // Shared-memory, socket, RDMA or mixed edges: a one-element ring AllReduce on two internal words.  No
        // rank's kernel completes before every rank's kernel has started, which is what a barrier promises.
        if (barrier_words_.data() == nullptr) barrier_words_ = RawDeviceBuffer(device_, 2 * sizeof(float), true);
        float* words = static_cast<float*>(barrier_words_.data());
        run_ring(CollectiveKind::AllReduce, words, words + 1, 1, DType::Float, RedOp::Sum, stream);
        return;
    }
    order_after_previous(stream);
    CUDA_CHECK_THROW(dev::launch_barrier(dev_, 1, stream));
}

void* Communicator::Impl::symmetric_alloc(std::size_t bytes) {
    check_async_error();
    NANO_REQUIRE_ARG(bytes > 0, "symmetric allocation must not be empty");
    NANO_REQUIRE(nvlink_path_, "symmetric memory needs GPU peer-to-peer transport on every edge");
    SymmetricMemory::Options options;
    options.want_multicast = multicast_available();
    options.zero = true;
    heap_.push_back(SymmetricMemory::create(*bootstrap_, fds_.get(), device_, bytes, options));
    return heap_.back()->local();
}

void Communicator::Impl::register_buffer(void* ptr, std::size_t bytes) {
    check_async_error();
    NANO_REQUIRE(nvlink_path_, "buffer registration needs GPU peer-to-peer transport on every edge");
    NANO_REQUIRE_ARG(find_symmetric(ptr, 1) == nullptr, "register: the buffer already lies inside symmetric or registered memory");
    heap_.push_back(SymmetricMemory::adopt(*bootstrap_, device_, ptr, bytes));
}

void Communicator::Impl::symmetric_free(void* ptr) {
    for (auto it = heap_.begin(); it != heap_.end(); ++it) {
        if ((*it)->local() == ptr) {
            CUDA_CHECK_THROW(cudaSetDevice(device_));
            CUDA_CHECK_THROW(cudaDeviceSynchronize());
            // Peers may still be mid-kernel on this memory: agree that everyone is done first.
            bootstrap_->barrier();
            heap_.erase(it);
            return;
        }
    }
    throw std::invalid_argument("symmetric_free: pointer was not returned by symmetric_alloc");
}

void* Communicator::Impl::peer_pointer(const void* ptr, int peer) const {
    NANO_REQUIRE_ARG(peer >= 0 && peer < nranks_, "peer rank %d out of range", peer);
    SymmetricMemory* seg = find_symmetric(ptr, 1);
    NANO_REQUIRE_ARG(seg != nullptr, "pointer is not inside symmetric memory of this communicator");
    const std::size_t off = static_cast<const char*>(ptr) - static_cast<const char*>(seg->local());
    return static_cast<char*>(seg->peer(peer)) + off;
}

void* Communicator::Impl::multicast_pointer(const void* ptr) const {
    SymmetricMemory* seg = find_symmetric(ptr, 1);
    NANO_REQUIRE_ARG(seg != nullptr, "pointer is not inside symmetric memory of this communicator");
    if (seg->multicast() == nullptr) return nullptr;
    const std::size_t off = static_cast<const char*>(ptr) - static_cast<const char*>(seg->local());
    return static_cast<char*>(seg->multicast()) + off;
}

TransportKind Communicator::Impl::edge_transport(int source) const {
    NANO_REQUIRE_ARG(source >= 0 && source < nranks_, "edge source rank %d outside 0..%d", source, nranks_ - 1);
    return plan_.edge_kinds[static_cast<std::size_t>(source)];
}

bool Communicator::Impl::edge_uses_gdr(int source) const {
    NANO_REQUIRE_ARG(source >= 0 && source < nranks_, "edge source rank %d outside 0..%d", source, nranks_ - 1);
    return ring_ != nullptr && ring_->edge_uses_gdr(source);
}

// ------------------------------------------------------------------------------------------------
// Public forwarding layer.
Communicator::Communicator(std::unique_ptr<Impl> impl) : impl_(std::move(impl)) {}
Communicator::Communicator(Communicator&&) noexcept = default;
Communicator& Communicator::operator=(Communicator&&) noexcept = default;
Communicator::~Communicator() = default;

namespace {
// NANO_NCCL_DEBUG=trace: what was asked for and which kernel family took it, one line per call.
void trace_call(const Communicator::Impl& impl, const char* what, std::size_t count, DType dtype, const char* op) {
    if (impl.debug_level_ < 2) return;
    std::fprintf(stderr, "nano_nccl[%d]: %s count=%zu dtype=%s op=%s -> %s (zero-copy calls so far %llu)\n", impl.rank_, what,
                 count, dtype_name(dtype), op, algo_name(impl.last_algo_),
                 static_cast<unsigned long long>(impl.stats_.zero_copy));
}
}  // namespace

void Communicator::all_reduce(const AllReduceArgs& args) {
    impl_->all_reduce(args);
    trace_call(*impl_, "all_reduce", args.count, args.dtype, redop_name(args.redop));
}
void Communicator::reduce_scatter(const ReduceScatterArgs& args) {
    impl_->reduce_scatter(args);
    trace_call(*impl_, "reduce_scatter", args.recv_count, args.dtype, redop_name(args.redop));
}
void Communicator::all_gather(const AllGatherArgs& args) {
    impl_->all_gather(args);
    trace_call(*impl_, "all_gather", args.send_count, args.dtype, "-");
}
void Communicator::check_async_error() const { impl_->check_async_error(); }
int Communicator::local_rank_count() const noexcept { return 1; }
int Communicator::global_rank_count() const noexcept { return impl_->nranks_; }
TransportKind Communicator::transport() const noexcept { return impl_->plan_.resolved_kind(); }
TransportKind Communicator::edge_transport(int s) const { return impl_->edge_transport(s); }
bool Communicator::edge_uses_gdr(int s) const { return impl_->edge_uses_gdr(s); }
int Communicator::rank() const noexcept { return impl_->rank_; }
int Communicator::device() const noexcept { return impl_->device_; }
bool Communicator::multicast_available() const noexcept { return impl_->multicast_available(); }
bool Communicator::relaxed_validation() const noexcept { return impl_->relaxed_validation_ || impl_->config_relaxed(); }
void* Communicator::symmetric_alloc(std::size_t bytes) { return impl_->symmetric_alloc(bytes); }
void Communicator::symmetric_free(void* ptr) { impl_->symmetric_free(ptr); }
void Communicator::register_buffer(void* ptr, std::size_t bytes) { impl_->register_buffer(ptr, bytes); }
void Communicator::deregister_buffer(void* ptr) { impl_->symmetric_free(ptr); }
bool Communicator::is_symmetric(const void* ptr, std::size_t bytes) const noexcept {
    return impl_->find_symmetric(ptr, bytes) != nullptr;
}
void* Communicator::peer_pointer(const void* ptr, int peer) const { return impl_->peer_pointer(ptr, peer); }
void* Communicator::multicast_pointer(const void* ptr) const { return impl_->multicast_pointer(ptr); }
void Communicator::barrier(cudaStream_t stream) { impl_->barrier(stream); }
void Communicator::set_algo(AlgoKind algo) noexcept { impl_->tuner_->set_forced_algo(algo); }
void Communicator::set_grid_override(int ctas) noexcept { impl_->tuner_->set_grid_override(ctas); }
AlgoKind Communicator::last_algo() const noexcept { return impl_->last_algo_; }
CommunicatorStats Communicator::stats() const noexcept { return impl_->stats_; }
Bootstrap& Communicator::bootstrap() const { return *impl_->bootstrap_; }

namespace collective {
std::unique_ptr<Communicator> CommunicatorFactory::create(std::shared_ptr<Bootstrap> bootstrap,
                                                          const CommunicatorConfig& config) {
    auto impl = std::make_unique<Communicator::Impl>(std::move(bootstrap), config);
    return std::unique_ptr<Communicator>(new Communicator(std::move(impl)));
}
Communicator::Impl& CommunicatorFactory::impl(Communicator& c) { return *c.impl_; }
}  // namespace collective

std::unique_ptr<Communicator> create_communicator(std::shared_ptr<Bootstrap> bootstrap,
                                                  const CommunicatorConfig& config) {
    return collective::CommunicatorFactory::create(std::move(bootstrap), config);
}

}  // namespace nano_nccl
