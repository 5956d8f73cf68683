// Launchers and tile geometry of the software-pipelined kernels (kernels/pipelined.cuh).
#include "kernels/dispatch.cuh"
#include "kernels/pipelined.cuh"

#include <algorithm>

namespace nano_nccl::dev {

// A CTA should walk at least four tiles, or the pipeline never fills; a tile below 32 KiB spends its time on
// flags.  So the grid shrinks until a CTA's region holds four such tiles (never below 16 CTAs, which still
// drive most of a link), and the tile is a quarter of the region, capped by what a pipeline buffer holds.
Geometry make_pipe_geometry(Family family, std::size_t count, std::size_t elem_size, int nranks, int max_grid,
                            std::size_t tile_bytes_hint) {
    const std::size_t n = static_cast<std::size_t>(nranks);
    std::size_t cap = 0;       // largest tile (bytes of the tiled dimension) a pipeline buffer holds
    std::size_t floor_tile = 32 * 1024;
    switch (family) {
        case Family::ArTwoShot: cap = std::min<std::size_t>(256 * 1024, (kPipeBufBytes / 2) / n / 16 * 16 * n); break;
        case Family::ArNvls: cap = 512 * 1024; break;
        default:  // ReduceScatter / AllGather: a buffer holds one tile per rank
            cap = kPipeBufBytes / n / 256 * 256;
            floor_tile = std::max<std::size_t>(8 * 1024, floor_tile / n);
            break;
    }
    const std::size_t bytes = count * elem_size;
    int grid = std::max(1, std::min(max_grid, kMaxBlocks));
    while (grid > 16 && bytes / static_cast<std::size_t>(grid) < 4 * floor_tile) grid /= 2;
    std::size_t tile = tile_bytes_hint != 0 ? tile_bytes_hint : std::max(floor_tile, bytes / static_cast<std::size_t>(grid) / 4);
    tile = std::min(tile, cap);
    return make_geometry(family, count, elem_size, nranks, grid, /*allow_skew=*/false, tile);
}

cudaError_t launch_ar_twoshot_pipe(const CommDev& c, const void* src, void* dst, std::size_t count, DType dtype, RedOp op,
                                   bool multicast, const Geometry& g, cudaStream_t stream) {
    if (static_cast<std::size_t>(c.nranks) * g.slot_bytes > kPipeBufBytes / 2) return cudaErrorInvalidValue;
    return dispatch_dtype(dtype, [&](auto t) {
        using T = decltype(t);
        return dispatch_op(op, [&](auto o) {
            constexpr RedOp Op = decltype(o)::value;
            if (multicast) {
                ar_twoshot_pipe_kernel<T, Op, true><<<g.grid, kCollectiveThreads, 0, stream>>>(
                    c, static_cast<const T*>(src), static_cast<T*>(dst), count, g);
            } else {
                ar_twoshot_pipe_kernel<T, Op, false><<<g.grid, kCollectiveThreads, 0, stream>>>(
                    c, static_cast<const T*>(src), static_cast<T*>(dst), count, g);
            }
            return cudaGetLastError();
        });
    });
}

cudaError_t launch_ar_nvls_pipe(const CommDev& c, const void* src, void* dst, std::size_t count, DType dtype, RedOp op,
                                const Geometry& g, cudaStream_t stream) {
    if (c.stage_mc == nullptr || !(op == RedOp::Sum || op == RedOp::Avg)) return cudaErrorInvalidValue;
    if (g.tile_elems * dtype_size(dtype) > kPipeBufBytes) return cudaErrorInvalidValue;
    return dispatch_dtype(dtype, [&](auto t) {
        using T = decltype(t);
        if (op == RedOp::Sum) {
            ar_nvls_pipe_kernel<T, RedOp::Sum><<<g.grid, kCollectiveThreads, 0, stream>>>(
                c, static_cast<const T*>(src), static_cast<T*>(dst), count, g);
        } else {
            ar_nvls_pipe_kernel<T, RedOp::Avg><<<g.grid, kCollectiveThreads, 0, stream>>>(
                c, static_cast<const T*>(src), static_cast<T*>(dst), count, g);
        }
        return cudaGetLastError();
    });
}

cudaError_t launch_rs_pipe(const CommDev& c, const void* src, void* dst, std::size_t recv_count, DType dtype, RedOp op,
                           const Geometry& g, cudaStream_t stream) {
    if (static_cast<std::size_t>(c.nranks) * g.slot_bytes > kPipeBufBytes) return cudaErrorInvalidValue;
    return dispatch_dtype(dtype, [&](auto t) {
        using T = decltype(t);
        return dispatch_op(op, [&](auto o) {
            constexpr RedOp Op = decltype(o)::value;
            rs_pipe_kernel<T, Op><<<g.grid, kCollectiveThreads, 0, stream>>>(
                c, static_cast<const T*>(src), static_cast<T*>(dst), recv_count, g);
            return cudaGetLastError();
        });
    });
}

cudaError_t launch_ag_pipe(const CommDev& c, const void* src, void* dst, std::size_t send_count, DType dtype,
                           bool multicast, const Geometry& g, cudaStream_t stream) {
    if (static_cast<std::size_t>(c.nranks) * g.slot_bytes > kPipeBufBytes) return cudaErrorInvalidValue;
    auto go = [&](auto t) {
        using T = decltype(t);
        if (multicast) {
            ag_pipe_kernel<T, true><<<g.grid, kCollectiveThreads, 0, stream>>>(
                c, static_cast<const T*>(src), static_cast<T*>(dst), send_count, g);
        } else {
            ag_pipe_kernel<T, false><<<g.grid, kCollectiveThreads, 0, stream>>>(
                c, static_cast<const T*>(src), static_cast<T*>(dst), send_count, g);
        }
        return cudaGetLastError();
    };
    return dtype == DType::Float ? go(float{}) : go(__half{});  // AllGather moves bits: only the element width matters
}

}  // namespace nano_nccl::dev
