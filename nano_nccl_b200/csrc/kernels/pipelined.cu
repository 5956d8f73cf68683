// Launchers and tile geometry of the software-pipelined kernels (kernels/pipelined.cuh).
#include "kernels/dispatch.cuh"
#include "kernels/pipelined.cuh"

#include <algorithm>

namespace nano_nccl::dev {

// The tile is what a CTA moves per iteration; the depth D is how many iterations separate a tile's stages.
// A signal (fence + flag flight) takes some 10 us on a busy link; an iteration moves one tile at the CTA's share of
// the link (about 4.5 GB/s with 128 CTAs), i.e. 32 KiB in about 7 us.  So: tiles of a sixteenth of the CTA's
// region, at least 16 KiB (8 KiB per rank for ReduceScatter / AllGather, whose staging holds one tile per rank)
// and at most what a buffer holds; D = 4 unless a hint says otherwise; the grid shrinks (never below 16 CTAs)
// until a region holds at least eight such tiles.
Geometry make_pipe_geometry(Family family, std::size_t count, std::size_t elem_size, int nranks, int max_grid,
                            std::size_t tile_bytes_hint, int depth_hint) {
    const std::size_t n = static_cast<std::size_t>(nranks);
    const int depth = std::max(1, std::min(depth_hint != 0 ? depth_hint : 4, kMaxPipeDepth));
    const std::size_t buf = pipe_buf_bytes(depth);
    std::size_t cap = 0;       // largest tile (bytes of the tiled dimension) a pipeline buffer holds
    std::size_t floor_tile = 16 * 1024;
    switch (family) {
        case Family::ArTwoShot: cap = (buf / 2) / n / 16 * 16 * n; break;   // scatter half + gather half, N slots each
        case Family::ArNvls: cap = buf / (16 * n) * (16 * n); break;
        default:  // ReduceScatter / AllGather: a buffer holds one tile per rank
            cap = buf / n / 256 * 256;
            floor_tile = std::max<std::size_t>(4 * 1024, floor_tile / n);
            break;
    }
    const std::size_t bytes = count * elem_size;
    int grid = std::max(1, std::min(max_grid, kMaxBlocks));
    while (grid > 16 && bytes / static_cast<std::size_t>(grid) < 8 * floor_tile) grid /= 2;
    std::size_t tile = tile_bytes_hint != 0 ? tile_bytes_hint : std::max(floor_tile, bytes / static_cast<std::size_t>(grid) / 16);
    tile = std::min(tile, cap);
    Geometry g = make_geometry(family, count, elem_size, nranks, grid, /*allow_skew=*/false, tile);
    g.depth = depth;
    return g;
}

cudaError_t launch_ar_twoshot_pipe(const CommDev& c, const void* src, void* dst, std::size_t count, DType dtype, RedOp op,
                                   bool multicast, const Geometry& g, cudaStream_t stream) {
    if (g.depth < 1 || g.depth > kMaxPipeDepth || static_cast<std::size_t>(c.nranks) * g.slot_bytes > pipe_buf_bytes(g.depth) / 2) return cudaErrorInvalidValue;
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
    if (g.depth < 1 || g.depth > kMaxPipeDepth || g.tile_elems * dtype_size(dtype) > pipe_buf_bytes(g.depth)) return cudaErrorInvalidValue;
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
    if (g.depth < 1 || g.depth > kMaxPipeDepth || static_cast<std::size_t>(c.nranks) * g.slot_bytes > pipe_buf_bytes(g.depth)) return cudaErrorInvalidValue;
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
    if (g.depth < 1 || g.depth > kMaxPipeDepth || static_cast<std::size_t>(c.nranks) * g.slot_bytes > pipe_buf_bytes(g.depth)) return cudaErrorInvalidValue;
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
