// nano_nccl_all_reduce_local_noalloc: the one-shot AllReduce of the single-GPU emulation with all
// scratch memory in a file-scope device array, for callers that may not allocate device memory.
// See include/nano_nccl/nano_nccl_noalloc.h for the contract.  No counterpart in the reference.
#include "capi/c_api_internal.h"
#include "kernels/dispatch.cuh"
#include "nano_nccl/nano_nccl_noalloc.h"

#include <mutex>

namespace {

using namespace nano_nccl;
using namespace nano_nccl::dev;

// Layout of the scratch array:
//   [0, kControlBytes)                     control: block counters and status words of every rank,
//                                          then the signal pads of every rank (cleared per call)
//   [kControlBytes, ...)                   staging of rank r, one CTA's worth (two 1 MiB halves)
constexpr int kRanksMax = NANO_NCCL_NOALLOC_MAX_RANKS;
constexpr std::size_t kMiscBytes = 64 * 1024;  // counters + status words
constexpr std::size_t kControlBytes = kMiscBytes + kRanksMax * kPadBytes;
constexpr std::size_t kScratchBytes = kControlBytes + kRanksMax * kBlockStageBytes;
static_assert(kScratchBytes == NANO_NCCL_NOALLOC_SCRATCH_BYTES, "the header states the scratch size");
static_assert(kRanksMax <= kMaxRanks, "rank limit");
static_assert(kRanksMax * (sizeof(BlockState) * kMaxBlocks + 64) <= kMiscBytes, "control area");

// In host code this name is only a handle for cudaGetSymbolAddress; device code may use it directly.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// Device address of the scratch array on the current device (looked up once per device).
cudaError_t scratch_for_current_device(unsigned char** out) {
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return err;
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_addr[device] == nullptr) {
        void* p = nullptr;
        err = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (err != cudaSuccess) return err;
        g_scratch_addr[device] = static_cast<unsigned char*>(p);
    }
    *out = g_scratch_addr[device];
    return cudaSuccess;
}

// The emulation context travels as a kernel parameter: no upload buffer is needed.
template <typename T, RedOp Op>
__global__ void __launch_bounds__(kCollectiveThreads, 1)
ar_oneshot_noalloc_kernel(const __grid_constant__ EmuRanks e, std::size_t count, const Geometry g) {
    const int r = blockIdx.y;
    ar_oneshot_body<T, Op, false>(e.ctx[r], static_cast<const T*>(e.src[r]), static_cast<T*>(e.dst[r]), count, g);
}

}  // namespace

extern "C" nano_nccl_status_t nano_nccl_all_reduce_local_noalloc(const void* const* srcs, void* const* dsts,
                                                                 int nranks, size_t count, nano_nccl_dtype_t dtype,
                                                                 nano_nccl_redop_t redop, cudaStream_t stream) {
    using namespace nano_nccl::c_api;
    begin_call();
    if (srcs == nullptr || dsts == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "srcs and dsts must be non-null");
    if (nranks < 1 || nranks > kRanksMax) {
        return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "nranks is outside 1..NANO_NCCL_NOALLOC_MAX_RANKS (8)");
    }
    if (count < 1 || count > NANO_NCCL_NOALLOC_MAX_COUNT) {
        return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT,
                    "count is outside 1..NANO_NCCL_NOALLOC_MAX_COUNT (4194304 elements): the fixed scratch array "
                    "of this entry point is sized for that; use the allocating entry points for larger buffers");
    }
    DType dt;
    RedOp op;
    if (!to_dtype(dtype, &dt)) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "unknown dtype");
    if (!to_redop(redop, &op)) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "unknown reduction operator");
    for (int r = 0; r < nranks; ++r) {
        if (srcs[r] == nullptr || dsts[r] == nullptr || srcs[r] == dsts[r]) {
            return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "every rank needs distinct non-null source and destination buffers");
        }
    }
    unsigned char* scratch = nullptr;
    if (scratch_for_current_device(&scratch) != cudaSuccess) {
        cudaGetLastError();
        return fail(NANO_NCCL_STATUS_ERROR, "cudaGetSymbolAddress of the scratch array failed on the current device");
    }
    // Counters, status words and pads start from zero in every call; staging needs no clearing
    // (every byte that is read was written earlier in the same call).
    if (cudaMemsetAsync(scratch, 0, kControlBytes, stream) != cudaSuccess) {
        cudaGetLastError();
        return fail(NANO_NCCL_STATUS_ERROR, "clearing the control part of the scratch array failed");
    }
    EmuRanks e{};
    for (int r = 0; r < nranks; ++r) {
        CommDev& c = e.ctx[r];
        c.rank = r;
        c.nranks = nranks;
        for (int p = 0; p < nranks; ++p) {
            c.pad[p] = reinterpret_cast<std::uint32_t*>(scratch + kMiscBytes + static_cast<std::size_t>(p) * kPadBytes);
            // one CTA per rank: stage_offset() of block 0 is 0, so the rank's staging starts here
            c.stage[p] = reinterpret_cast<char*>(scratch + kControlBytes + static_cast<std::size_t>(p) * kBlockStageBytes);
        }
        c.stage_mc = nullptr;
        c.state = reinterpret_cast<BlockState*>(scratch + static_cast<std::size_t>(r) * sizeof(BlockState) * kMaxBlocks);
        std::uint32_t* status = reinterpret_cast<std::uint32_t*>(scratch + kRanksMax * sizeof(BlockState) * kMaxBlocks);
        c.status = status + 8 * r;
        c.abort_flag = status + 8 * kRanksMax;  // never raised: stays zero
        c.timeout_ns = 5'000'000'000ull;
        e.src[r] = srcs[r];
        e.dst[r] = dsts[r];
    }
    // One CTA per rank walks all tiles of the message.
    Geometry g = make_geometry(Family::ArOneShot, count, dtype_size(dt), nranks, /*max_grid=*/1);
    const dim3 grid(1, static_cast<unsigned>(nranks));
    std::size_t count_arg = count;
    void* params[] = {&e, &count_arg, &g};
    const cudaError_t err = dispatch_dtype(dt, [&](auto t) {
        using T = decltype(t);
        return dispatch_op(op, [&](auto o) {
            constexpr RedOp Op = decltype(o)::value;
            // cooperative: the nranks CTAs wait on one another and must all be resident
            return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(ar_oneshot_noalloc_kernel<T, Op>), grid,
                                               dim3(kCollectiveThreads), params, 0, stream);
        });
    });
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(NANO_NCCL_STATUS_ERROR, cudaGetErrorString(err));
    }
    return NANO_NCCL_STATUS_SUCCESS;
}

extern "C" nano_nccl_status_t nano_nccl_all_reduce_local_noalloc_status(cudaStream_t stream, uint32_t words[4]) {
    using namespace nano_nccl::c_api;
    begin_call();
    if (words == nullptr) return fail(NANO_NCCL_STATUS_INVALID_ARGUMENT, "words must be non-null");
    words[0] = words[1] = words[2] = words[3] = 0;
    unsigned char* scratch = nullptr;
    if (scratch_for_current_device(&scratch) != cudaSuccess) {
        cudaGetLastError();
        return fail(NANO_NCCL_STATUS_ERROR, "cudaGetSymbolAddress of the scratch array failed on the current device");
    }
    if (cudaStreamSynchronize(stream) != cudaSuccess) {
        cudaGetLastError();
        return fail(NANO_NCCL_STATUS_ERROR, "waiting for the stream failed");
    }
    // eight status words per rank, on the stack: no allocation here either
    std::uint32_t all[8 * kRanksMax] = {};
    const unsigned char* status = scratch + kRanksMax * sizeof(BlockState) * kMaxBlocks;
    if (cudaMemcpy(all, status, sizeof(all), cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError();
        return fail(NANO_NCCL_STATUS_ERROR, "reading the status words failed");
    }
    for (int r = 0; r < kRanksMax; ++r) {
        if (all[8 * r] != 0) {
            for (int k = 0; k < 4; ++k) words[k] = all[8 * r + k];
            return fail(NANO_NCCL_STATUS_ERROR,
                        "the last allocation-free AllReduce on this device ended early: a bounded wait ran out; its outputs are incomplete");
        }
    }
    return NANO_NCCL_STATUS_SUCCESS;
}
