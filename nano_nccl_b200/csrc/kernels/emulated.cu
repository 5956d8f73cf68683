#include "kernels/emulated.h"

#include "core/env.h"

#include "core/buffer.h"
#include "core/error.h"
#include "kernels/dispatch.cuh"
#include "kernels/ll_collectives.cuh"
#include "kernels/pipelined.cuh"

#include <vector>

namespace nano_nccl::dev {

struct EmulatedCluster::State {
    std::vector<RawDeviceBuffer> arenas;
    std::vector<RawDeviceBuffer> states;
    MappedU32Array status;  // 8 words per rank
    MappedU32Array abort_word;
    RawDeviceBuffer ranks_dev;  // EmuRanks
    EmuRanks ranks_host{};
    // flag-in-data kernels (NANO_NCCL_LL_MAX_BYTES > 0 when the cluster is created)
    std::vector<RawDeviceBuffer> ll_arenas;
    RawDeviceBuffer ll_dev;     // LLDev
    std::size_t ll_max_bytes = 0;
    // software-pipelined kernels for messages of at least this size (NANO_NCCL_PIPE_MIN_BYTES when the cluster is created)
    std::size_t pipe_min_bytes = 0;
    std::size_t pipe_tile_bytes = 0;
    int pipe_depth = 0;
};

namespace {
__global__ void __launch_bounds__(kCollectiveThreads, 1) lonely_barrier_kernel(CommDev c) {
    std::uint32_t epoch = c.state[blockIdx.x].epoch;
    const std::uint32_t seq = c.state[blockIdx.x].seq;
    block_barrier(c, epoch, 9);
    // The epoch is not persisted: the barrier did not complete.
    save_state(c, epoch - 1, seq);
}

template <typename Kernel, typename... Args>
void launch_cooperative_smem(Kernel kernel, dim3 grid, std::size_t smem, cudaStream_t stream, Args... args) {
    int per_sm = 0, sms = 0, device = 0;
    CUDA_CHECK_THROW(cudaGetDevice(&device));
    if (smem > 48 * 1024) {
        CUDA_CHECK_THROW(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    }
    CUDA_CHECK_THROW(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kCollectiveThreads, smem));
    CUDA_CHECK_THROW(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    NANO_REQUIRE(static_cast<long>(grid.x) * grid.y <= static_cast<long>(per_sm) * sms,
                 "emulated cluster: %u x %u blocks cannot be co-resident (%d per SM x %d SMs)", grid.x,
                 grid.y, per_sm, sms);
    void* params[] = {static_cast<void*>(&args)...};
    CUDA_CHECK_THROW(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), grid,
                                                 dim3(kCollectiveThreads), params, smem, stream));
}
template <typename Kernel, typename... Args>
void launch_cooperative(Kernel kernel, dim3 grid, cudaStream_t stream, Args... args) {
    launch_cooperative_smem(kernel, grid, 0, stream, args...);
}
}  // namespace

EmulatedCluster::EmulatedCluster(int device, int nranks, std::int64_t timeout_us)
    : s_(new State()), device_(device), nranks_(nranks) {
    NANO_REQUIRE_ARG(nranks >= 1 && nranks <= kMaxRanks, "emulated cluster: 1..%d ranks", kMaxRanks);
    CUDA_CHECK_THROW(cudaSetDevice(device));
    s_->status = MappedU32Array(8 * kMaxRanks);
    s_->abort_word = MappedU32Array(8);
    for (int r = 0; r < nranks; ++r) {
        s_->arenas.emplace_back(device, kArenaBytes, true);
        s_->states.emplace_back(device, sizeof(BlockState) * kMaxBlocks, true);
    }
    for (int r = 0; r < nranks; ++r) {
        CommDev& c = s_->ranks_host.ctx[r];
        c = CommDev{};
        c.rank = r;
        c.nranks = nranks;
        for (int p = 0; p < nranks; ++p) {
            char* base = static_cast<char*>(s_->arenas[p].data());
            c.pad[p] = reinterpret_cast<std::uint32_t*>(base);
            c.stage[p] = base + kPadBytes;
        }
        c.stage_mc = nullptr;
        c.state = static_cast<BlockState*>(s_->states[r].data());
        c.status = s_->status.device() + 8 * r;
        c.abort_flag = s_->abort_word.device();
        c.timeout_ns = static_cast<unsigned long long>(timeout_us) * 1000ull;
    }
    s_->ranks_dev = RawDeviceBuffer(device, sizeof(EmuRanks));
    s_->ll_max_bytes = static_cast<std::size_t>(env::integer("NANO_NCCL_LL_MAX_BYTES", 0, 0, 16 << 20));
    s_->pipe_min_bytes = static_cast<std::size_t>(env::integer("NANO_NCCL_PIPE_MIN_BYTES", 0, 0, 1ll << 40));
    s_->pipe_tile_bytes = static_cast<std::size_t>(env::integer("NANO_NCCL_PIPE_TILE_BYTES", 0, 0, 1 << 20));
    s_->pipe_depth = static_cast<int>(env::integer("NANO_NCCL_PIPE_DEPTH", 0, 0, kMaxPipeDepth));
    if (s_->ll_max_bytes != 0) {
        LLDev l{};
        for (int r = 0; r < nranks; ++r) {
            s_->ll_arenas.emplace_back(device, kLLArenaBytes, true);
            l.stage[r] = static_cast<char*>(s_->ll_arenas[r].data());
        }
        s_->ll_dev = RawDeviceBuffer(device, sizeof(LLDev));
        CUDA_CHECK_THROW(cudaMemcpy(s_->ll_dev.data(), &l, sizeof(LLDev), cudaMemcpyHostToDevice));
    }
}

EmulatedCluster::~EmulatedCluster() {
    cudaSetDevice(device_);
    cudaDeviceSynchronize();
}

static void upload(EmuRanks& host, RawDeviceBuffer& dev, const void* const* srcs, void* const* dsts,
                   int nranks, cudaStream_t stream) {
    for (int r = 0; r < nranks; ++r) {
        host.src[r] = srcs[r];
        host.dst[r] = dsts[r];
    }
    // Synchronous small copy: the host struct is reused by the next call.
    CUDA_CHECK_THROW(cudaMemcpyAsync(dev.data(), &host, sizeof(EmuRanks), cudaMemcpyHostToDevice, stream));
    CUDA_CHECK_THROW(cudaStreamSynchronize(stream));
}

void EmulatedCluster::all_reduce(const void* const* srcs, void* const* dsts, std::size_t count, DType dtype,
                                 RedOp op, AlgoKind algo, int max_grid, cudaStream_t stream) {
    NANO_REQUIRE_ARG(algo == AlgoKind::OneShot || algo == AlgoKind::TwoShot,
                     "emulated cluster runs the oneshot and twoshot variants only");
    CUDA_CHECK_THROW(cudaSetDevice(device_));
    upload(s_->ranks_host, s_->ranks_dev, srcs, dsts, nranks_, stream);
    const Family fam = algo == AlgoKind::OneShot ? Family::ArOneShot : Family::ArTwoShot;
    const bool ll = algo == AlgoKind::OneShot && s_->ll_max_bytes != 0 && count * dtype_size(dtype) <= s_->ll_max_bytes;
    const bool pipe = algo == AlgoKind::TwoShot && s_->pipe_min_bytes != 0 && count * dtype_size(dtype) >= s_->pipe_min_bytes;
    const Geometry g = pipe ? make_pipe_geometry(fam, count, dtype_size(dtype), nranks_, max_grid, s_->pipe_tile_bytes, s_->pipe_depth)
                            : make_geometry(fam, count, dtype_size(dtype), nranks_, max_grid, !ll, ll ? ll_tile_cap_bytes(nranks_) : 0);
    const EmuRanks* e = static_cast<const EmuRanks*>(s_->ranks_dev.data());
    const LLDev* l = static_cast<const LLDev*>(s_->ll_dev.data());
    const dim3 grid(g.grid, nranks_);
    CUDA_CHECK_THROW(dispatch_dtype(dtype, [&](auto t) {
        using T = decltype(t);
        return dispatch_op(op, [&](auto o) {
            constexpr RedOp Op = decltype(o)::value;
            if (pipe) {
                launch_cooperative(ar_twoshot_pipe_emu_kernel<T, Op>, grid, stream, e, count, g);
            } else if (ll) {
                launch_cooperative(ar_oneshot_ll_emu_kernel<T, Op>, grid, stream, e, l, count, g);
            } else if (algo == AlgoKind::OneShot) {
                launch_cooperative(ar_oneshot_emu_kernel<T, Op>, grid, stream, e, count, g);
            } else {
                launch_cooperative(ar_twoshot_emu_kernel<T, Op>, grid, stream, e, count, g);
            }
            return cudaGetLastError();
        });
    }));
}

void EmulatedCluster::reduce_scatter(const void* const* srcs, void* const* dsts, std::size_t recv_count,
                                     DType dtype, RedOp op, int max_grid, cudaStream_t stream) {
    CUDA_CHECK_THROW(cudaSetDevice(device_));
    upload(s_->ranks_host, s_->ranks_dev, srcs, dsts, nranks_, stream);
    const bool ll = s_->ll_max_bytes != 0 && recv_count * dtype_size(dtype) * nranks_ <= s_->ll_max_bytes;
    const bool pipe = s_->pipe_min_bytes != 0 && recv_count * dtype_size(dtype) * nranks_ >= s_->pipe_min_bytes;
    const Geometry g = pipe ? make_pipe_geometry(Family::ReduceScatter, recv_count, dtype_size(dtype), nranks_, max_grid, s_->pipe_tile_bytes, s_->pipe_depth)
                            : make_geometry(Family::ReduceScatter, recv_count, dtype_size(dtype), nranks_, max_grid, true,
                                            ll ? ll_tile_cap_bytes(nranks_) : 0);
    const EmuRanks* e = static_cast<const EmuRanks*>(s_->ranks_dev.data());
    const LLDev* l = static_cast<const LLDev*>(s_->ll_dev.data());
    const dim3 grid(g.grid, nranks_);
    CUDA_CHECK_THROW(dispatch_dtype(dtype, [&](auto t) {
        using T = decltype(t);
        return dispatch_op(op, [&](auto o) {
            constexpr RedOp Op = decltype(o)::value;
            if (pipe) launch_cooperative(rs_pipe_emu_kernel<T, Op>, grid, stream, e, recv_count, g);
            else if (ll) launch_cooperative(rs_ll_emu_kernel<T, Op>, grid, stream, e, l, recv_count, g);
            else launch_cooperative(rs_push_emu_kernel<T, Op>, grid, stream, e, recv_count, g);
            return cudaGetLastError();
        });
    }));
}

void EmulatedCluster::all_gather(const void* const* srcs, void* const* dsts, std::size_t send_count,
                                 DType dtype, int max_grid, cudaStream_t stream) {
    CUDA_CHECK_THROW(cudaSetDevice(device_));
    upload(s_->ranks_host, s_->ranks_dev, srcs, dsts, nranks_, stream);
    const bool ll = s_->ll_max_bytes != 0 && send_count * dtype_size(dtype) * nranks_ <= s_->ll_max_bytes;
    const bool pipe = s_->pipe_min_bytes != 0 && send_count * dtype_size(dtype) * nranks_ >= s_->pipe_min_bytes &&
                      !env::flag("NANO_NCCL_PUSH_TMA", false);
    const Geometry g = pipe ? make_pipe_geometry(Family::AllGather, send_count, dtype_size(dtype), nranks_, max_grid, s_->pipe_tile_bytes, s_->pipe_depth)
                            : make_geometry(Family::AllGather, send_count, dtype_size(dtype), nranks_, max_grid, true,
                                            ll ? ll_tile_cap_bytes(nranks_) : 0);
    const EmuRanks* e = static_cast<const EmuRanks*>(s_->ranks_dev.data());
    const dim3 grid(g.grid, nranks_);
    if (pipe) {
        if (dtype == DType::Float) launch_cooperative(ag_pipe_emu_kernel<float>, grid, stream, e, send_count, g);
        else launch_cooperative(ag_pipe_emu_kernel<__half>, grid, stream, e, send_count, g);
        CUDA_CHECK_THROW(cudaGetLastError());
        return;
    }
    if (ll) {
        const LLDev* l = static_cast<const LLDev*>(s_->ll_dev.data());
        if (dtype == DType::Float) launch_cooperative(ag_ll_emu_kernel<float>, grid, stream, e, l, send_count, g);
        else launch_cooperative(ag_ll_emu_kernel<__half>, grid, stream, e, l, send_count, g);
        CUDA_CHECK_THROW(cudaGetLastError());
        return;
    }
    // NANO_NCCL_PUSH_TMA=1 selects the variant whose pushes are TMA bulk copies, when the buffers allow it
    bool tma = env::flag("NANO_NCCL_PUSH_TMA", false) && (send_count * dtype_size(dtype)) % 16 == 0;
    for (int r = 0; r < nranks_ && tma; ++r) {
        tma = reinterpret_cast<std::uintptr_t>(srcs[r]) % 16 == 0 && reinterpret_cast<std::uintptr_t>(dsts[r]) % 16 == 0;
    }
    if (tma) {
        if (dtype == DType::Float) {
            launch_cooperative_smem(ag_push_tma_emu_kernel<float>, grid, kPipeSmemBytes, stream, e, send_count, g);
        } else {
            launch_cooperative_smem(ag_push_tma_emu_kernel<__half>, grid, kPipeSmemBytes, stream, e, send_count, g);
        }
    } else if (dtype == DType::Float) {
        launch_cooperative(ag_push_emu_kernel<float>, grid, stream, e, send_count, g);
    } else {
        launch_cooperative(ag_push_emu_kernel<__half>, grid, stream, e, send_count, g);
    }
    CUDA_CHECK_THROW(cudaGetLastError());
}

void EmulatedCluster::lonely_barrier(int rank, cudaStream_t stream) {
    NANO_REQUIRE_ARG(rank >= 0 && rank < nranks_, "rank out of range");
    CUDA_CHECK_THROW(cudaSetDevice(device_));
    lonely_barrier_kernel<<<1, kCollectiveThreads, 0, stream>>>(s_->ranks_host.ctx[rank]);
    CUDA_CHECK_THROW(cudaGetLastError());
}

void EmulatedCluster::status(int rank, std::uint32_t out[4]) const {
    const volatile std::uint32_t* w = s_->status.host() + 8 * rank;
    for (int i = 0; i < 4; ++i) out[i] = w[i];
}

void EmulatedCluster::clear_status() {
    for (std::size_t i = 0; i < s_->status.size(); ++i) s_->status.host()[i] = 0;
}

void EmulatedCluster::set_abort(bool on) { s_->abort_word.host()[0] = on ? 1u : 0u; }

}  // namespace nano_nccl::dev
