// Host-side entry points of the collective kernels: runtime (dtype, redop) -> template dispatch.
// Each returns the cudaError_t of the launch.  Parity: reference
// src/collective/all_reduce/communicator.cu:63-85 (the three kernel launchers).
#pragma once

#include "kernels/device_context.h"

#include <cuda_runtime.h>

namespace nano_nccl::dev {

// How a message is cut: CTA b owns the contiguous region [b * region_elems, (b+1) * region_elems)
// and walks it tile by tile.  With `skew`, odd CTAs shift their tile boundaries by half a tile
// (first tile half-size), so that at any moment about half of the CTAs are in the egress-heavy
// push phase while the others are in the ingress-heavy reduce / broadcast phase, instead of all
// CTAs of all GPUs marching through the phases together.
#if defined(__CUDACC__)
#define NANO_GEOM_HD_EARLY __host__ __device__ inline
#else
#define NANO_GEOM_HD_EARLY inline
#endif

struct Geometry {
    int grid = 1;                   // CTAs
    std::size_t region_elems = 0;   // elements per CTA (multiple of the tile unit)
    std::size_t tile_elems = 0;     // elements per tile (multiple of nranks * vector width, even number of units)
    int iters = 1;                  // tiles each CTA walks (padding tiles are empty)
    std::size_t slot_bytes = 0;     // staging bytes reserved per source rank (or per sub-slice)
    int skew = 0;
    int depth = 0;                  // pipelined kernels: iterations between a tile's stages (buffers = 2 * depth + 1)
};

// Pipelined kernels: a CTA's 2 MiB of staging cut into 2 * depth + 1 buffers (multiples of 1 KiB).
constexpr int kMaxPipeDepth = 8;
NANO_GEOM_HD_EARLY std::size_t pipe_buf_bytes(int depth) {
    return kBlockStageBytes / static_cast<std::size_t>(2 * depth + 1) / 1024 * 1024;
}

#if defined(__CUDACC__)
#define NANO_GEOM_HD __host__ __device__ inline
#else
#define NANO_GEOM_HD inline
#endif

// Tile `it` of CTA `block`: first element and length (0 for a padding iteration).
NANO_GEOM_HD void tile_range_of(const Geometry& g, std::size_t count, unsigned block, int it, std::size_t* t0,
                                std::size_t* n) {
    const std::size_t rb = static_cast<std::size_t>(block) * g.region_elems;
    *t0 = count;
    *n = 0;
    if (rb >= count) return;
    const std::size_t re = (count - rb < g.region_elems) ? count : rb + g.region_elems;
    const std::size_t T = g.tile_elems;
    std::size_t s, e;
    if (g.skew != 0 && (block & 1u) != 0u) {
        // odd CTAs: half tile first, then full tiles shifted by half a tile
        s = it == 0 ? 0 : static_cast<std::size_t>(it) * T - T / 2;
        e = it == 0 ? T / 2 : s + T;
    } else {
        s = static_cast<std::size_t>(it) * T;
        e = s + T;
    }
    s += rb;
    e += rb;
    if (s >= re) return;
    *t0 = s;
    *n = (e < re ? e : re) - s;
}

enum class Family { ArOneShot, ArTwoShot, ArNvls, ReduceScatter, AllGather };

// Largest tile (in bytes) the staging layout of a family allows for `nranks`.
std::size_t max_tile_bytes(Family family, int nranks);
// Cuts `count` elements of `elem_size` bytes into tiles for at most `max_grid` CTAs.
// `tile_cap_bytes` > 0 caps the tile below what the staging half allows, so that a CTA walks several
// tiles and the phases of different CTAs drift apart (tuning knob NANO_NCCL_TILE_BYTES).
Geometry make_geometry(Family family, std::size_t count, std::size_t elem_size, int nranks,
                       int max_grid, bool allow_skew = true, std::size_t tile_cap_bytes = 0);

cudaError_t launch_ar_oneshot(const CommDev& c, const void* src, void* dst, std::size_t count,
                              DType dtype, RedOp op, bool multicast, const Geometry& g,
                              cudaStream_t stream);
cudaError_t launch_ar_twoshot(const CommDev& c, const void* src, void* dst, std::size_t count,
                              DType dtype, RedOp op, bool multicast, const Geometry& g,
                              cudaStream_t stream);
cudaError_t launch_ar_nvls(const CommDev& c, const void* src, void* dst, std::size_t count,
                           DType dtype, RedOp op, const Geometry& g, cudaStream_t stream);
// src_mc / dst_mc: multicast aliases of symmetric buffers; bytes must be a multiple of 16.
cudaError_t launch_ar_nvls_symm(const CommDev& c, const void* src_mc, void* dst_mc,
                                std::size_t bytes, DType dtype, RedOp op, int grid,
                                cudaStream_t stream);
// Zero-copy AllReduce over peer pointers of symmetric buffers (no multicast needed).
// src_peers / dst_peers: nranks views of the same buffers; bytes % 16 == 0.
// Zero-copy ReduceScatter: `src_mc` is the multicast view of a symmetric input of nranks chunks of
// `chunk_bytes` (a multiple of 16); `dst` is this rank's ordinary, 16-byte aligned output.  Sum / Avg.
cudaError_t launch_rs_nvls_symm(const CommDev& c, const void* src_mc, void* dst, std::size_t chunk_bytes,
                                DType dtype, RedOp op, int grid, cudaStream_t stream);
// Zero-copy AllGather: `src` is this rank's ordinary, 16-byte aligned chunk; the symmetric output is
// given as every rank's view (`dst_peers`) and, when `dst_mc` is not null, its multicast view.
cudaError_t launch_ag_symm(const CommDev& c, const void* src, void* const* dst_peers, void* dst_mc,
                           std::size_t chunk_bytes, int grid, cudaStream_t stream);
cudaError_t launch_ar_symm_p2p(const CommDev& c, const void* const* src_peers, void* const* dst_peers,
                               std::size_t bytes, DType dtype, RedOp op, bool one_shot, int grid,
                               cudaStream_t stream);
cudaError_t launch_rs_push(const CommDev& c, const void* src, void* dst, std::size_t recv_count,
                           DType dtype, RedOp op, const Geometry& g, cudaStream_t stream);
cudaError_t launch_ag_push(const CommDev& c, const void* src, void* dst, std::size_t send_count,
                           DType dtype, bool multicast, const Geometry& g, cudaStream_t stream);
// AllGather whose pushes are TMA bulk copies; cudaErrorInvalidValue when the buffers are not 16-byte
// aligned or the chunk is not a multiple of 16 bytes (the caller then uses launch_ag_push).
cudaError_t launch_ag_push_tma(const CommDev& c, const void* src, void* dst, std::size_t send_count, DType dtype,
                               const Geometry& g, cudaStream_t stream);
// Flag-in-data (LL) kernels for small messages: no barrier, twice the bytes on the wire.  `g` must come from
// make_geometry with tile_cap_bytes = ll_tile_cap_bytes(nranks).
std::size_t ll_tile_cap_bytes(int nranks);
cudaError_t launch_ar_oneshot_ll(const CommDev& c, const LLDev& l, const void* src, void* dst, std::size_t count,
                                 DType dtype, RedOp op, bool multicast, const Geometry& g, cudaStream_t stream);
cudaError_t launch_rs_ll(const CommDev& c, const LLDev& l, const void* src, void* dst, std::size_t recv_count,
                         DType dtype, RedOp op, const Geometry& g, cudaStream_t stream);
cudaError_t launch_ag_ll(const CommDev& c, const LLDev& l, const void* src, void* dst, std::size_t send_count,
                         DType dtype, bool multicast, const Geometry& g, cudaStream_t stream);
cudaError_t launch_barrier(const CommDev& c, int grid, cudaStream_t stream);

// Software-pipelined forms for large messages (kernels/pipelined.cuh): a CTA keeps three tiles in flight and
// waits only for signals that are one iteration old.  `g` must come from make_pipe_geometry.
Geometry make_pipe_geometry(Family family, std::size_t count, std::size_t elem_size, int nranks, int max_grid,
                            std::size_t tile_bytes_hint = 0, int depth_hint = 0);
cudaError_t launch_ar_twoshot_pipe(const CommDev& c, const void* src, void* dst, std::size_t count, DType dtype, RedOp op,
                                   bool multicast, const Geometry& g, cudaStream_t stream);
cudaError_t launch_ar_nvls_pipe(const CommDev& c, const void* src, void* dst, std::size_t count, DType dtype, RedOp op,
                                const Geometry& g, cudaStream_t stream);
cudaError_t launch_rs_pipe(const CommDev& c, const void* src, void* dst, std::size_t recv_count, DType dtype, RedOp op,
                           const Geometry& g, cudaStream_t stream);
cudaError_t launch_ag_pipe(const CommDev& c, const void* src, void* dst, std::size_t send_count, DType dtype,
                           bool multicast, const Geometry& g, cudaStream_t stream);

// Copies `bytes` (a multiple of 16) from `src` to each of `ndst` destinations, all 16-byte aligned, with
// untiled TMA bulk copies through `stages` (3..16) shared-memory stages of `chunk_bytes` per CTA
// (kernels/bulk_copy.cu).  `device_error` is a zeroed device word that becomes 1 if a wait ran out.
cudaError_t launch_bulk_push(const void* src, void* const* dsts, int ndst, std::size_t bytes, int ctas,
                             int chunk_bytes, int stages, int* device_error, cudaStream_t stream);
// The same copy with 16-byte vector loads and stores from `ctas` blocks of threads.
cudaError_t launch_sm_push(const void* src, void* const* dsts, int ndst, std::size_t bytes, int ctas,
                           cudaStream_t stream);

}  // namespace nano_nccl::dev
