// The NVLink 5 / NVSwitch collective kernels (device code).  Every kernel is tile-pipelined per
// CTA: CTA b handles tiles b, b+G, b+2G, ... of the message and synchronises only with CTA b of
// the other GPUs, so at any moment different CTAs are in different phases and local HBM copies,
// NVLink pushes and reductions overlap across the grid without a grid-wide phase barrier.
//
// Kernels (T = float / __half / __nv_bfloat16, Op = Sum / Avg / Max / Min):
//   ar_oneshot_kernel   push whole tile to every peer (P2P stores or one multimem.st), one
//                       barrier, every rank reduces all N copies locally in rank order.
//   ar_twoshot_kernel   push sub-slice j to its owner j, barrier, owner reduces in fp32 and
//                       broadcasts the result (P2P stores or multimem.st), barrier, copy out.
//   ar_nvls_kernel      copy tile into the multicast-bound staging, barrier, owner slice:
//                       multimem.ld_reduce (in-switch sum) -> scale -> multimem.st, barrier,
//                       copy out.  Sum / Avg only.
//   ar_nvls_symm_kernel the same on caller-owned symmetric buffers: no staging copies at all.
//   rs_push_kernel      push chunk j of the tile to rank j, barrier, reduce into the dense output.
//   ag_push_kernel      push own tile to everyone, barrier, copy the peers' tiles out.
//
// Parity: these replace ring_simple_kernel / ring_simple_reduce_scatter_kernel /
// ring_simple_all_gather_kernel (reference src/kernels/ring_simple_kernel.cuh:1466-1735) on an
// NVSwitch box: 1 or 2 hops instead of 2(N-1), up to 148 CTAs moving data instead of <= 4, fp32
// accumulation, the avg scale and the output cast fused into the final combine.  Max / Min keep
// the reference's NaN rule (a NaN operand wins) because they never go through the switch ALU.
#pragma once

#include "kernels/bulk_pipe.cuh"
#include "kernels/launch.h"
#include "kernels/prims.cuh"

namespace nano_nccl::dev {

// Elements [i, i+EPV) of p, zero beyond n.  `aligned` says p is 16-byte aligned (i is a multiple
// of the vector width, so p+i then is too).
template <typename T>
__device__ __forceinline__ Vec16 load_guarded(const T* p, std::size_t i, std::size_t n, bool aligned) {
    constexpr int kE = ElemsPerVec<T>::value;
    if (aligned && i + kE <= n) return ld_vec_stream(p + i);
    Vec16 v{{0u, 0u, 0u, 0u}};
    T* e = reinterpret_cast<T*>(&v);
#pragma unroll
    for (int k = 0; k < kE; ++k) {
        if (i + k < n) e[k] = p[i + k];
    }
    return v;
}

template <typename T>
__device__ __forceinline__ void store_guarded(T* p, std::size_t i, std::size_t n, bool aligned,
                                              const Vec16& v) {
    constexpr int kE = ElemsPerVec<T>::value;
    if (aligned && i + kE <= n) {
        st_vec(p + i, v);
        return;
    }
    const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
    for (int k = 0; k < kE; ++k) {
        if (i + k < n) p[i + k] = e[k];
    }
}

__device__ __forceinline__ void tile_range(std::size_t count, const Geometry& g, int it, std::size_t* t0,
                                           std::size_t* n) {
    tile_range_of(g, count, blockIdx.x, it, t0, n);
}

__device__ __forceinline__ std::size_t stage_offset(int half) {
    return static_cast<std::size_t>(blockIdx.x) * kBlockStageBytes + static_cast<std::size_t>(half) * kHalfBytes;
}

__device__ __forceinline__ void save_state(const CommDev& c, std::uint32_t epoch, std::uint32_t seq) {
    if (threadIdx.x == 0) {
        c.state[blockIdx.x].epoch = epoch;
        c.state[blockIdx.x].seq = seq;
    }
}

// Every kernel re-checks on the device, once per tile, that the staging footprint the host computed fits
// this block's staging half: `slots` slots of `slot_bytes` inside `area_bytes`, of which a slot uses
// `used_bytes`.  A violation is recorded as kStatusBadArgument {slots, used_bytes / 16} and the block leaves
// before touching staging (its peers' waits then run out and report the same call).  The answer is uniform
// over the block; the check is a handful of integer operations per tile, so it is part of every build (the
// stand-in for a memory checker, which the target machines do not offer).
__device__ __forceinline__ bool tile_fits(const CommDev& c, std::size_t used_bytes, std::size_t slot_bytes, int slots,
                                          std::size_t area_bytes) {
    const bool ok = blockIdx.x < static_cast<unsigned>(kMaxBlocks) && slot_bytes % 16 == 0 && used_bytes <= slot_bytes &&
                    static_cast<std::size_t>(slots) * slot_bytes <= area_bytes;
    if (!ok && threadIdx.x == 0) report_status(c, kStatusBadArgument, slots, static_cast<int>(used_bytes >> 4));
    return ok;
}

// Largest sub-slice of a tile of n elements split over N owners, in bytes of whole 16-byte vectors.
template <typename T>
__device__ __forceinline__ std::size_t max_split_bytes(std::size_t n, int N) {
    constexpr int kE = ElemsPerVec<T>::value;
    std::size_t most = 0;
    for (int j = 0; j < N; ++j) {
        const std::size_t len = split_begin(n, N, j + 1, kE) - split_begin(n, N, j, kE);
        most = len > most ? len : most;
    }
    return (most + kE - 1) / kE * 16;
}

constexpr int kBatch = 8;  // independent 16-byte accesses each thread keeps in flight

// ------------------------------------------------------------------------------------------------
// One-shot AllReduce.  slot_bytes = bytes reserved per source rank inside a staging half.
template <typename T, RedOp Op, bool kMc>
__device__ __forceinline__ void
ar_oneshot_body(const CommDev& c, const T* src, T* dst, std::size_t count,
                  const Geometry g) {
    constexpr int kE = ElemsPerVec<T>::value;
    std::uint32_t epoch = c.state[blockIdx.x].epoch;
    std::uint32_t seq = c.state[blockIdx.x].seq;
    const float inv = 1.0f / static_cast<float>(c.nranks);
    for (int it = 0; it < g.iters; ++it, ++seq) {
        std::size_t t0, n;
        tile_range(count, g, it, &t0, &n);
        const std::size_t nvec = (n + kE - 1) / kE;
        if (!tile_fits(c, nvec * 16, g.slot_bytes, c.nranks, kHalfBytes)) break;
        const std::size_t off = stage_offset(seq & 1u);
        const T* s = src + t0;
        T* d = dst + t0;
        const bool s_al = aligned16(s), d_al = aligned16(d);
        // push my copy of the tile into slot[rank] on every rank
        for (std::size_t v0 = threadIdx.x; v0 < nvec; v0 += kBatch * blockDim.x) {
            Vec16 x[kBatch];
#pragma unroll
            for (int k = 0; k < kBatch; ++k) {
                const std::size_t v = v0 + k * blockDim.x;
                if (v < nvec) x[k] = load_guarded(s, v * kE, n, s_al);
            }
#pragma unroll
            for (int k = 0; k < kBatch; ++k) {
                const std::size_t v = v0 + k * blockDim.x;
                if (v < nvec) {
                    const std::size_t o = off + c.rank * g.slot_bytes + v * 16;
                    if constexpr (kMc) {
                        multimem_st(c.stage_mc + o, x[k]);
                    } else {
                        for (int i = 1; i < c.nranks; ++i) {
                            st_vec(c.stage[(c.rank + i) % c.nranks] + o, x[k]);
                        }
                    }
                }
            }
        }
        if (!block_barrier(c, epoch, 1)) break;
        // every rank reduces all copies in rank order: results are bit-identical on all ranks
        const char* mine = c.stage[c.rank] + off;
        for (std::size_t v = threadIdx.x; v < nvec; v += blockDim.x) {
            // My own contribution comes straight from the input: a multimem.st to my own copy
            // has no flag that orders it before this read.
            Acc<T> acc;
            for (int r = 0; r < c.nranks; ++r) {
                const Vec16 x = (r == c.rank) ? load_guarded(s, v * kE, n, s_al)
                                              : ld_vec_volatile(mine + r * g.slot_bytes + v * 16);
                if (r == 0) acc = unpack<T>(x); else combine<Op, T>(acc, unpack<T>(x));
            }
            finish<Op, T>(acc, inv);
            store_guarded(d, v * kE, n, d_al, pack<T>(acc));
        }
    }
    save_state(c, epoch, seq);
}

// ------------------------------------------------------------------------------------------------
// Two-shot AllReduce.  slot_bytes = bytes reserved per rank sub-slice; scatter area is the first
// half of the staging half, gather area the second.
template <typename T, RedOp Op, bool kMc>
__device__ __forceinline__ void
ar_twoshot_body(const CommDev& c, const T* src, T* dst, std::size_t count,
                  const Geometry g) {
    constexpr int kE = ElemsPerVec<T>::value;
    constexpr std::size_t kGatherOff = kHalfBytes / 2;
    std::uint32_t epoch = c.state[blockIdx.x].epoch;
    std::uint32_t seq = c.state[blockIdx.x].seq;
    const float inv = 1.0f / static_cast<float>(c.nranks);
    const int N = c.nranks;
    for (int it = 0; it < g.iters; ++it, ++seq) {
        std::size_t t0, n;
        tile_range(count, g, it, &t0, &n);
        if (!tile_fits(c, max_split_bytes<T>(n, N), g.slot_bytes, N, kGatherOff)) break;
        const std::size_t off = stage_offset(seq & 1u);
        const T* s = src + t0;
        T* d = dst + t0;
        const bool s_al = aligned16(s), d_al = aligned16(d);
        // phase 1: scatter sub-slice j of my tile to rank j
        for (int i = 1; i < N; ++i) {
            const int j = (c.rank + i) % N;
            const std::size_t b = split_begin(n, N, j, kE), e = split_begin(n, N, j + 1, kE);
            const std::size_t len = e - b, nvec = (len + kE - 1) / kE;
            char* out = c.stage[j] + off + c.rank * g.slot_bytes;
            for (std::size_t v0 = threadIdx.x; v0 < nvec; v0 += kBatch * blockDim.x) {
                Vec16 x[kBatch];
#pragma unroll
                for (int k = 0; k < kBatch; ++k) {
                    const std::size_t v = v0 + k * blockDim.x;
                    if (v < nvec) x[k] = load_guarded(s + b, v * kE, len, s_al);
                }
#pragma unroll
                for (int k = 0; k < kBatch; ++k) {
                    const std::size_t v = v0 + k * blockDim.x;
                    if (v < nvec) st_vec(out + v * 16, x[k]);
                }
            }
        }
        if (!block_barrier(c, epoch, 1)) break;
        // phase 2: reduce my sub-slice (fp32, rank order), write it to my output and to everyone
        {
            const std::size_t b = split_begin(n, N, c.rank, kE), e = split_begin(n, N, c.rank + 1, kE);
            const std::size_t len = e - b, nvec = (len + kE - 1) / kE;
            const char* in = c.stage[c.rank] + off;
            const std::size_t go = off + kGatherOff + c.rank * g.slot_bytes;
            for (std::size_t v = threadIdx.x; v < nvec; v += blockDim.x) {
                Acc<T> acc;
                for (int r = 0; r < N; ++r) {
                    const Vec16 x = (r == c.rank) ? load_guarded(s + b, v * kE, len, s_al)
                                                  : ld_vec_volatile(in + r * g.slot_bytes + v * 16);
                    if (r == 0) acc = unpack<T>(x); else combine<Op, T>(acc, unpack<T>(x));
                }
                finish<Op, T>(acc, inv);
                const Vec16 y = pack<T>(acc);
                store_guarded(d + b, v * kE, len, d_al, y);
                if constexpr (kMc) {
                    multimem_st(c.stage_mc + go + v * 16, y);
                } else {
                    for (int i = 1; i < N; ++i) st_vec(c.stage[(c.rank + i) % N] + go + v * 16, y);
                }
            }
        }
        if (!block_barrier(c, epoch, 2)) break;
        // phase 3: copy the other owners' results out of my gather area
        for (int i = 1; i < N; ++i) {
            const int j = (c.rank + i) % N;
            const std::size_t b = split_begin(n, N, j, kE), e = split_begin(n, N, j + 1, kE);
            const std::size_t len = e - b, nvec = (len + kE - 1) / kE;
            const char* in = c.stage[c.rank] + off + kGatherOff + j * g.slot_bytes;
            for (std::size_t v0 = threadIdx.x; v0 < nvec; v0 += kBatch * blockDim.x) {
                Vec16 x[kBatch];
#pragma unroll
                for (int k = 0; k < kBatch; ++k) {
                    const std::size_t v = v0 + k * blockDim.x;
                    if (v < nvec) x[k] = ld_vec_volatile(in + v * 16);
                }
#pragma unroll
                for (int k = 0; k < kBatch; ++k) {
                    const std::size_t v = v0 + k * blockDim.x;
                    if (v < nvec) store_guarded(d + b, v * kE, len, d_al, x[k]);
                }
            }
        }
    }
    save_state(c, epoch, seq);
}

// ------------------------------------------------------------------------------------------------
// NVLS AllReduce through the staging arena (arbitrary user buffers).  Sum / Avg.
template <typename T, RedOp Op>
__device__ __forceinline__ void
ar_nvls_body(const CommDev& c, const T* src, T* dst, std::size_t count,
               const Geometry g) {
    static_assert(Op == RedOp::Sum || Op == RedOp::Avg, "the switch only adds");
    constexpr int kE = ElemsPerVec<T>::value;
    std::uint32_t epoch = c.state[blockIdx.x].epoch;
    std::uint32_t seq = c.state[blockIdx.x].seq;
    const float inv = 1.0f / static_cast<float>(c.nranks);
    const int N = c.nranks;
    for (int it = 0; it < g.iters; ++it, ++seq) {
        std::size_t t0, n;
        tile_range(count, g, it, &t0, &n);
        const std::size_t nvec = (n + kE - 1) / kE;
        if (!tile_fits(c, nvec * 16, kHalfBytes, 1, kHalfBytes)) break;
        const std::size_t off = stage_offset(seq & 1u);
        const T* s = src + t0;
        T* d = dst + t0;
        const bool s_al = aligned16(s), d_al = aligned16(d);
        char* mine = c.stage[c.rank] + off;
        // phase 1: bring the tile into multicast-bound memory
        for (std::size_t v0 = threadIdx.x; v0 < nvec; v0 += kBatch * blockDim.x) {
            Vec16 x[kBatch];
#pragma unroll
            for (int k = 0; k < kBatch; ++k) {
                const std::size_t v = v0 + k * blockDim.x;
                if (v < nvec) x[k] = load_guarded(s, v * kE, n, s_al);
            }
#pragma unroll
            for (int k = 0; k < kBatch; ++k) {
                const std::size_t v = v0 + k * blockDim.x;
                if (v < nvec) st_vec(mine + v * 16, x[k]);
            }
        }
        if (!block_barrier(c, epoch, 1)) break;
        // phase 2: in-switch reduction of my slice, broadcast of the result
        const std::size_t b = split_begin(n, N, c.rank, kE), e = split_begin(n, N, c.rank + 1, kE);
        {
            const std::size_t vb = (b + kE - 1) / kE, ve = (e + kE - 1) / kE;  // b == n when the slice is empty
            for (std::size_t v0 = vb + threadIdx.x; v0 < ve; v0 += kBatch * blockDim.x) {
                Vec16 x[kBatch];
#pragma unroll
                for (int k = 0; k < kBatch; ++k) {
                    const std::size_t v = v0 + k * blockDim.x;
                    if (v < ve) x[k] = multimem_ld_reduce_add<T>(c.stage_mc + off + v * 16);
                }
#pragma unroll
                for (int k = 0; k < kBatch; ++k) {
                    const std::size_t v = v0 + k * blockDim.x;
                    if (v < ve) {
                        if constexpr (Op == RedOp::Avg) {
                            Acc<T> a = unpack<T>(x[k]);
                            finish<Op, T>(a, inv);
                            x[k] = pack<T>(a);
                        }
                        multimem_st(c.stage_mc + off + v * 16, x[k]);
                        store_guarded(d, v * kE, n, d_al, x[k]);
                    }
                }
            }
        }
        if (!block_barrier(c, epoch, 2)) break;
        // phase 3: copy out everything I did not produce myself
        {
            const std::size_t vb = (b + kE - 1) / kE, ve = (e + kE - 1) / kE;  // b == n when the slice is empty
            for (std::size_t v0 = threadIdx.x; v0 < nvec; v0 += kBatch * blockDim.x) {
                Vec16 x[kBatch];
#pragma unroll
                for (int k = 0; k < kBatch; ++k) {
                    const std::size_t v = v0 + k * blockDim.x;
                    if (v < nvec && (v < vb || v >= ve)) x[k] = ld_vec_volatile(mine + v * 16);
                }
#pragma unroll
                for (int k = 0; k < kBatch; ++k) {
                    const std::size_t v = v0 + k * blockDim.x;
                    if (v < nvec && (v < vb || v >= ve)) store_guarded(d, v * kE, n, d_al, x[k]);
                }
            }
        }
    }
    save_state(c, epoch, seq);
}

// ------------------------------------------------------------------------------------------------
// NVLS AllReduce on caller-owned symmetric buffers: src_mc / dst_mc are the multicast aliases of
// the input and output.  Requires 16-byte aligned buffers and count * sizeof(T) % 16 == 0.
// In place (src == dst) is allowed: each vector is read and written by exactly one thread.
template <typename T, RedOp Op>
__device__ __forceinline__ void
ar_nvls_symm_body(const CommDev& c, const char* src_mc, char* dst_mc,
                    std::size_t nvec_total) {
    static_assert(Op == RedOp::Sum || Op == RedOp::Avg, "the switch only adds");
    std::uint32_t epoch = c.state[blockIdx.x].epoch;
    const std::uint32_t seq = c.state[blockIdx.x].seq;
    const float inv = 1.0f / static_cast<float>(c.nranks);
    // All peers have produced their inputs once their same-index block arrives here.
    if (block_barrier(c, epoch, 1)) {
        // Rank r owns vectors [r*per, (r+1)*per); the grid strides over that range.
        const std::size_t per = (nvec_total + c.nranks - 1) / c.nranks;
        const std::size_t vb = per * c.rank < nvec_total ? per * c.rank : nvec_total;
        const std::size_t ve = vb + per < nvec_total ? vb + per : nvec_total;
        const std::size_t stride = static_cast<std::size_t>(gridDim.x) * blockDim.x;
        for (std::size_t v0 = vb + blockIdx.x * blockDim.x + threadIdx.x; v0 < ve; v0 += kBatch * stride) {
            Vec16 x[kBatch];
#pragma unroll
            for (int k = 0; k < kBatch; ++k) {
                const std::size_t v = v0 + k * stride;
                if (v < ve) x[k] = multimem_ld_reduce_add<T>(src_mc + v * 16);
            }
#pragma unroll
            for (int k = 0; k < kBatch; ++k) {
                const std::size_t v = v0 + k * stride;
                if (v < ve) {
                    if constexpr (Op == RedOp::Avg) {
                        Acc<T> a = unpack<T>(x[k]);
                        finish<Op, T>(a, inv);
                        x[k] = pack<T>(a);
                    }
                    multimem_st(dst_mc + v * 16, x[k]);
                }
            }
        }
        // Results of all owners have landed (and nobody still reads my input) after this.
        block_barrier(c, epoch, 2);
    }
    save_state(c, epoch, seq);
}

// ------------------------------------------------------------------------------------------------
// ReduceScatter: `count` = recv_count; input chunk j (count elements) belongs to rank j.
template <typename T, RedOp Op>
__device__ __forceinline__ void
rs_push_body(const CommDev& c, const T* src, T* dst, std::size_t count,
               const Geometry g) {
    constexpr int kE = ElemsPerVec<T>::value;
    std::uint32_t epoch = c.state[blockIdx.x].epoch;
    std::uint32_t seq = c.state[blockIdx.x].seq;
    const float inv = 1.0f / static_cast<float>(c.nranks);
    const int N = c.nranks;
    for (int it = 0; it < g.iters; ++it, ++seq) {
        std::size_t t0, n;
        tile_range(count, g, it, &t0, &n);
        const std::size_t nvec = (n + kE - 1) / kE;
        if (!tile_fits(c, nvec * 16, g.slot_bytes, N, kHalfBytes)) break;
        const std::size_t off = stage_offset(seq & 1u);
        for (int i = 1; i < N; ++i) {
            const int j = (c.rank + i) % N;
            const T* s = src + static_cast<std::size_t>(j) * count + t0;
            const bool s_al = aligned16(s);
            char* out = c.stage[j] + off + c.rank * g.slot_bytes;
            for (std::size_t v0 = threadIdx.x; v0 < nvec; v0 += kBatch * blockDim.x) {
                Vec16 x[kBatch];
#pragma unroll
                for (int k = 0; k < kBatch; ++k) {
                    const std::size_t v = v0 + k * blockDim.x;
                    if (v < nvec) x[k] = load_guarded(s, v * kE, n, s_al);
                }
#pragma unroll
                for (int k = 0; k < kBatch; ++k) {
                    const std::size_t v = v0 + k * blockDim.x;
                    if (v < nvec) st_vec(out + v * 16, x[k]);
                }
            }
        }
        if (!block_barrier(c, epoch, 1)) break;
        const T* own = src + static_cast<std::size_t>(c.rank) * count + t0;
        const bool own_al = aligned16(own);
        T* d = dst + t0;
        const bool d_al = aligned16(d);
        const char* in = c.stage[c.rank] + off;
        for (std::size_t v = threadIdx.x; v < nvec; v += blockDim.x) {
            Acc<T> acc;
            for (int r = 0; r < N; ++r) {
                const Vec16 x = (r == c.rank) ? load_guarded(own, v * kE, n, own_al)
                                              : ld_vec_volatile(in + r * g.slot_bytes + v * 16);
                if (r == 0) acc = unpack<T>(x); else combine<Op, T>(acc, unpack<T>(x));
            }
            finish<Op, T>(acc, inv);
            store_guarded(d, v * kE, n, d_al, pack<T>(acc));
        }
    }
    save_state(c, epoch, seq);
}

// ------------------------------------------------------------------------------------------------
// AllGather: `count` = send_count; output is rank-major.  T only fixes the element width.
template <typename T, bool kMc>
__device__ __forceinline__ void
ag_push_body(const CommDev& c, const T* src, T* dst, std::size_t count,
               const Geometry g) {
    constexpr int kE = ElemsPerVec<T>::value;
    std::uint32_t epoch = c.state[blockIdx.x].epoch;
    std::uint32_t seq = c.state[blockIdx.x].seq;
    const int N = c.nranks;
    for (int it = 0; it < g.iters; ++it, ++seq) {
        std::size_t t0, n;
        tile_range(count, g, it, &t0, &n);
        const std::size_t nvec = (n + kE - 1) / kE;
        if (!tile_fits(c, nvec * 16, g.slot_bytes, N, kHalfBytes)) break;
        const std::size_t off = stage_offset(seq & 1u);
        const T* s = src + t0;
        const bool s_al = aligned16(s);
        T* own = dst + static_cast<std::size_t>(c.rank) * count + t0;
        const bool own_al = aligned16(own);
        for (std::size_t v0 = threadIdx.x; v0 < nvec; v0 += kBatch * blockDim.x) {
            Vec16 x[kBatch];
#pragma unroll
            for (int k = 0; k < kBatch; ++k) {
                const std::size_t v = v0 + k * blockDim.x;
                if (v < nvec) x[k] = load_guarded(s, v * kE, n, s_al);
            }
#pragma unroll
            for (int k = 0; k < kBatch; ++k) {
                const std::size_t v = v0 + k * blockDim.x;
                if (v < nvec) {
                    store_guarded(own, v * kE, n, own_al, x[k]);
                    const std::size_t o = off + c.rank * g.slot_bytes + v * 16;
                    if constexpr (kMc) {
                        multimem_st(c.stage_mc + o, x[k]);
                    } else {
                        for (int i = 1; i < N; ++i) st_vec(c.stage[(c.rank + i) % N] + o, x[k]);
                    }
                }
            }
        }
        if (!block_barrier(c, epoch, 1)) break;
        for (int i = 1; i < N; ++i) {
            const int j = (c.rank + i) % N;
            T* d = dst + static_cast<std::size_t>(j) * count + t0;
            const bool d_al = aligned16(d);
            const char* in = c.stage[c.rank] + off + j * g.slot_bytes;
            for (std::size_t v0 = threadIdx.x; v0 < nvec; v0 += kBatch * blockDim.x) {
                Vec16 x[kBatch];
#pragma unroll
                for (int k = 0; k < kBatch; ++k) {
                    const std::size_t v = v0 + k * blockDim.x;
                    if (v < nvec) x[k] = ld_vec_volatile(in + v * 16);
                }
#pragma unroll
                for (int k = 0; k < kBatch; ++k) {
                    const std::size_t v = v0 + k * blockDim.x;
                    if (v < nvec) store_guarded(d, v * kE, n, d_al, x[k]);
                }
            }
        }
    }
    save_state(c, epoch, seq);
}

// AllGather whose pushes are TMA bulk copies: per tile, thread 0 sends the tile into slot `rank` of
// every peer's staging and into this rank's own place in the output; the rest is ag_push_body (one
// barrier, then all threads copy the peers' tiles out of the local staging).  Needs 16-byte aligned
// src / dst and count * sizeof(T) a multiple of 16 (the launcher checks).
template <typename T>
__device__ __forceinline__ void
ag_push_tma_body(const CommDev& c, const T* src, T* dst, std::size_t count, const Geometry g, unsigned char* smem) {
    constexpr int kE = ElemsPerVec<T>::value;
    std::uint32_t epoch = c.state[blockIdx.x].epoch;
    std::uint32_t seq = c.state[blockIdx.x].seq;
    const int N = c.nranks;
    BulkPipe pipe;
    pipe_init(pipe, smem);
    __shared__ int push_failed;
    if (threadIdx.x == 0) push_failed = 0;
    __syncthreads();
    for (int it = 0; it < g.iters; ++it, ++seq) {
        std::size_t t0, n;
        tile_range(count, g, it, &t0, &n);
        const std::size_t nvec = (n + kE - 1) / kE;
        if (!tile_fits(c, nvec * 16, g.slot_bytes, N, kHalfBytes)) break;
        const std::size_t off = stage_offset(seq & 1u);
        if (threadIdx.x == 0 && n != 0) {
            char* targets[kMaxRanks];
            targets[0] = reinterpret_cast<char*>(dst + static_cast<std::size_t>(c.rank) * count + t0);
            for (int i = 1; i < N; ++i) targets[i] = c.stage[(c.rank + i) % N] + off + c.rank * g.slot_bytes;
            if (!pipe_push(pipe, reinterpret_cast<const char*>(src + t0), targets, N, n * sizeof(T))) {
                report_status(c, kStatusWaitTimeout, c.rank, 7);
                push_failed = 1;
            }
            __threadfence_system();
        }
        __syncthreads();
        if (push_failed != 0) break;
        if (!block_barrier(c, epoch, 1)) break;
        for (int i = 1; i < N; ++i) {
            const int j = (c.rank + i) % N;
            T* d = dst + static_cast<std::size_t>(j) * count + t0;
            const char* in = c.stage[c.rank] + off + j * g.slot_bytes;
            for (std::size_t v0 = threadIdx.x; v0 < nvec; v0 += kBatch * blockDim.x) {
                Vec16 x[kBatch];
#pragma unroll
                for (int k = 0; k < kBatch; ++k) {
                    const std::size_t v = v0 + k * blockDim.x;
                    if (v < nvec) x[k] = ld_vec_volatile(in + v * 16);
                }
#pragma unroll
                for (int k = 0; k < kBatch; ++k) {
                    const std::size_t v = v0 + k * blockDim.x;
                    if (v < nvec) st_vec(reinterpret_cast<char*>(d) + v * 16, x[k]);
                }
            }
        }
    }
    save_state(c, epoch, seq);
}

// ------------------------------------------------------------------------------------------------
// AllReduce on caller-owned symmetric buffers without multicast (peer loads and stores): zero
// staging.  src[r] / dst[r] are rank r's views of the same symmetric input / output.
// kOneShot: every rank loads all copies of the whole message and reduces them locally (small
// messages: one hop).  Otherwise two-shot: rank r reduces slice r from all peers' inputs and
// stores the result into every rank's output.  In place (src == dst) is safe in the two-shot
// form because slice r is read and written by rank r only; the one-shot form needs out-of-place
// buffers or relies on the trailing barrier with a distinct output.
// Requires 16-byte aligned buffers and a byte count that is a multiple of 16.
struct SymmPeers {
    const char* src[kMaxRanks];
    char* dst[kMaxRanks];
};

// kN: the rank count as a compile-time constant (2, 4, 8), or 0 for "whatever c.nranks says".  With kN known a
// thread keeps 16 / kN vectors of every rank in flight (16 loads of 16 bytes); a single vector per thread, as in the
// generic form, leaves a CTA at a few GB/s over NVLink, which matters when only a few CTAs may be spared for the
// reduction (gradient buckets beside a backward pass).
template <typename T, RedOp Op, bool kOneShot, int kN>
__device__ __forceinline__ void
ar_symm_p2p_body(const CommDev& c, const SymmPeers& p, std::size_t nvec_total) {
    std::uint32_t epoch = c.state[blockIdx.x].epoch;
    const std::uint32_t seq = c.state[blockIdx.x].seq;
    const float inv = 1.0f / static_cast<float>(c.nranks);
    const int N = kN != 0 ? kN : c.nranks;
    constexpr int kVecs = kN != 0 ? 16 / kN : 1;   // vectors per thread and pass
    constexpr int kR = kN != 0 ? kN : kMaxRanks;   // unrolled rank loop bound
    if (block_barrier(c, epoch, 1)) {  // every rank's input is complete
        std::size_t vb = 0, ve = nvec_total;
        if (!kOneShot) {
            const std::size_t per = (nvec_total + N - 1) / N;
            vb = per * c.rank < nvec_total ? per * c.rank : nvec_total;
            ve = vb + per < nvec_total ? vb + per : nvec_total;
        }
        const std::size_t stride = static_cast<std::size_t>(gridDim.x) * blockDim.x;
        for (std::size_t v0 = vb + blockIdx.x * blockDim.x + threadIdx.x; v0 < ve; v0 += kVecs * stride) {
            Vec16 x[kVecs][kR];
#pragma unroll
            for (int k = 0; k < kVecs; ++k) {
                const std::size_t v = v0 + k * stride;
#pragma unroll
                for (int r = 0; r < kR; ++r) {
                    if (r < N && v < ve) x[k][r] = ld_vec_volatile(p.src[r] + v * 16);  // all loads in flight together
                }
            }
#pragma unroll
            for (int k = 0; k < kVecs; ++k) {
                const std::size_t v = v0 + k * stride;
                if (v >= ve) continue;
                Acc<T> acc = unpack<T>(x[k][0]);
#pragma unroll
                for (int r = 1; r < kR; ++r) {
                    if (r < N) combine<Op, T>(acc, unpack<T>(x[k][r]));
                }
                finish<Op, T>(acc, inv);
                const Vec16 y = pack<T>(acc);
                if (kOneShot) {
                    st_vec(p.dst[c.rank] + v * 16, y);
                } else {
#pragma unroll
                    for (int i = 0; i < kR; ++i) {
                        if (i < N) st_vec(p.dst[(c.rank + i) % N] + v * 16, y);
                    }
                }
            }
        }
        // results have landed everywhere, and nobody still reads anybody's input
        block_barrier(c, epoch, 2);
    }
    save_state(c, epoch, seq);
}

// ------------------------------------------------------------------------------------------------
// ReduceScatter through the switch on a caller-owned symmetric input: rank r reads chunk r of the
// multicast view with multimem.ld_reduce (one load returns the sum over every rank's copy) and
// writes the dense result to its own, ordinary output.  No staging, no pushes; each GPU receives
// only its 1/N of the data.  Sum / Avg only.  `nvec_chunk` = 16-byte vectors per chunk.
template <typename T, RedOp Op>
__device__ __forceinline__ void
rs_nvls_symm_body(const CommDev& c, const char* src_mc, char* dst, std::size_t nvec_chunk) {
    static_assert(Op == RedOp::Sum || Op == RedOp::Avg, "the switch only adds");
    std::uint32_t epoch = c.state[blockIdx.x].epoch;
    const std::uint32_t seq = c.state[blockIdx.x].seq;
    const float inv = 1.0f / static_cast<float>(c.nranks);
    if (block_barrier(c, epoch, 1)) {  // every rank's input is complete
        const char* chunk = src_mc + static_cast<std::size_t>(c.rank) * nvec_chunk * 16;
        const std::size_t stride = static_cast<std::size_t>(gridDim.x) * blockDim.x;
        for (std::size_t v0 = blockIdx.x * blockDim.x + threadIdx.x; v0 < nvec_chunk; v0 += kBatch * stride) {
            Vec16 x[kBatch];
#pragma unroll
            for (int k = 0; k < kBatch; ++k) {
                const std::size_t v = v0 + k * stride;
                if (v < nvec_chunk) x[k] = multimem_ld_reduce_add<T>(chunk + v * 16);
            }
#pragma unroll
            for (int k = 0; k < kBatch; ++k) {
                const std::size_t v = v0 + k * stride;
                if (v < nvec_chunk) {
                    if constexpr (Op == RedOp::Avg) {
                        Acc<T> a = unpack<T>(x[k]);
                        finish<Op, T>(a, inv);
                        x[k] = pack<T>(a);
                    }
                    st_vec(dst + v * 16, x[k]);
                }
            }
        }
        // Nobody reads anybody's input any more once every rank has passed this point.
        block_barrier(c, epoch, 2);
    }
    save_state(c, epoch, seq);
}

// AllGather into a caller-owned symmetric output: every rank stores its chunk straight into slot
// `rank` of every rank's output (one multimem.st through the switch, or N plain stores), so nothing
// is staged and nothing is copied out.  The first barrier says that every rank has entered the call
// and its output may be written; the second that all chunks have landed.
template <bool kMc>
__device__ __forceinline__ void
ag_symm_body(const CommDev& c, const char* src, const SymmPeers& p, char* dst_mc, std::size_t nvec_chunk) {
    std::uint32_t epoch = c.state[blockIdx.x].epoch;
    const std::uint32_t seq = c.state[blockIdx.x].seq;
    const int N = c.nranks;
    if (block_barrier(c, epoch, 1)) {
        const std::size_t base = static_cast<std::size_t>(c.rank) * nvec_chunk * 16;
        const std::size_t stride = static_cast<std::size_t>(gridDim.x) * blockDim.x;
        for (std::size_t v0 = blockIdx.x * blockDim.x + threadIdx.x; v0 < nvec_chunk; v0 += kBatch * stride) {
            Vec16 x[kBatch];
#pragma unroll
            for (int k = 0; k < kBatch; ++k) {
                const std::size_t v = v0 + k * stride;
                if (v < nvec_chunk) x[k] = ld_vec_stream(src + v * 16);
            }
#pragma unroll
            for (int k = 0; k < kBatch; ++k) {
                const std::size_t v = v0 + k * stride;
                if (v < nvec_chunk) {
                    if constexpr (kMc) {
                        multimem_st(dst_mc + base + v * 16, x[k]);
                    } else {
#pragma unroll
                        for (int i = 0; i < kMaxRanks; ++i) {
                            if (i < N) st_vec(p.dst[(c.rank + i) % N] + base + v * 16, x[k]);
                        }
                    }
                }
            }
        }
        block_barrier(c, epoch, 2);
    }
    save_state(c, epoch, seq);
}

// ------------------------------------------------------------------------------------------------
// __global__ entry points.  `*_kernel`: one rank per GPU, context by value.  `*_emu_kernel`: all
// ranks of a communicator emulated on ONE GPU for testing (blockIdx.y is the rank; cooperative
// launch keeps every block resident, because blocks of different emulated ranks wait on one
// another).  The emulation runs exactly the device code of the P2P variants; multimem variants
// need a real multicast object and are only exercised on multi-GPU runs.
struct EmuRanks {
    CommDev ctx[kMaxRanks];
    const void* src[kMaxRanks];
    void* dst[kMaxRanks];
};

#define NANO_KERNEL __global__ void __launch_bounds__(kCollectiveThreads, 1)

template <typename T, RedOp Op, bool kMc>
NANO_KERNEL ar_oneshot_kernel(CommDev c, const T* src, T* dst, std::size_t count, const Geometry g) {
    ar_oneshot_body<T, Op, kMc>(c, src, dst, count, g);
}
template <typename T, RedOp Op>
NANO_KERNEL ar_oneshot_emu_kernel(const EmuRanks* e, std::size_t count, const Geometry g) {
    const int r = blockIdx.y;
    ar_oneshot_body<T, Op, false>(e->ctx[r], static_cast<const T*>(e->src[r]), static_cast<T*>(e->dst[r]), count, g);
}

template <typename T, RedOp Op, bool kMc>
NANO_KERNEL ar_twoshot_kernel(CommDev c, const T* src, T* dst, std::size_t count, const Geometry g) {
    ar_twoshot_body<T, Op, kMc>(c, src, dst, count, g);
}
template <typename T, RedOp Op>
NANO_KERNEL ar_twoshot_emu_kernel(const EmuRanks* e, std::size_t count, const Geometry g) {
    const int r = blockIdx.y;
    ar_twoshot_body<T, Op, false>(e->ctx[r], static_cast<const T*>(e->src[r]), static_cast<T*>(e->dst[r]), count, g);
}

template <typename T, RedOp Op>
NANO_KERNEL ar_nvls_kernel(CommDev c, const T* src, T* dst, std::size_t count, const Geometry g) {
    ar_nvls_body<T, Op>(c, src, dst, count, g);
}
template <typename T, RedOp Op>
NANO_KERNEL ar_nvls_symm_kernel(CommDev c, const char* src_mc, char* dst_mc, std::size_t nvec_total) {
    ar_nvls_symm_body<T, Op>(c, src_mc, dst_mc, nvec_total);
}

template <typename T>
NANO_KERNEL ag_push_tma_kernel(CommDev c, const T* src, T* dst, std::size_t count, const Geometry g) {
    extern __shared__ __align__(128) unsigned char pipe_smem[];
    ag_push_tma_body<T>(c, src, dst, count, g, pipe_smem);
}
template <typename T>
NANO_KERNEL ag_push_tma_emu_kernel(const EmuRanks* e, std::size_t count, const Geometry g) {
    extern __shared__ __align__(128) unsigned char pipe_smem[];
    const int r = blockIdx.y;
    ag_push_tma_body<T>(e->ctx[r], static_cast<const T*>(e->src[r]), static_cast<T*>(e->dst[r]), count, g, pipe_smem);
}

template <typename T, RedOp Op>
NANO_KERNEL rs_nvls_symm_kernel(CommDev c, const char* src_mc, char* dst, std::size_t nvec_chunk) {
    rs_nvls_symm_body<T, Op>(c, src_mc, dst, nvec_chunk);
}
template <bool kMc>
NANO_KERNEL ag_symm_kernel(CommDev c, const char* src, SymmPeers p, char* dst_mc, std::size_t nvec_chunk) {
    ag_symm_body<kMc>(c, src, p, dst_mc, nvec_chunk);
}

template <typename T, RedOp Op, bool kOneShot, int kN>
NANO_KERNEL ar_symm_p2p_kernel(CommDev c, SymmPeers p, std::size_t nvec_total) {
    ar_symm_p2p_body<T, Op, kOneShot, kN>(c, p, nvec_total);
}

template <typename T, RedOp Op>
NANO_KERNEL rs_push_kernel(CommDev c, const T* src, T* dst, std::size_t count, const Geometry g) {
    rs_push_body<T, Op>(c, src, dst, count, g);
}
template <typename T, RedOp Op>
NANO_KERNEL rs_push_emu_kernel(const EmuRanks* e, std::size_t count, const Geometry g) {
    const int r = blockIdx.y;
    rs_push_body<T, Op>(e->ctx[r], static_cast<const T*>(e->src[r]), static_cast<T*>(e->dst[r]), count, g);
}

template <typename T, bool kMc>
NANO_KERNEL ag_push_kernel(CommDev c, const T* src, T* dst, std::size_t count, const Geometry g) {
    ag_push_body<T, kMc>(c, src, dst, count, g);
}
template <typename T>
NANO_KERNEL ag_push_emu_kernel(const EmuRanks* e, std::size_t count, const Geometry g) {
    const int r = blockIdx.y;
    ag_push_body<T, false>(e->ctx[r], static_cast<const T*>(e->src[r]), static_cast<T*>(e->dst[r]), count, g);
}

}  // namespace nano_nccl::dev
