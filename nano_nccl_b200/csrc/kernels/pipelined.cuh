// Software-pipelined forms of the NVLink collective kernels for large messages.
//
// The plain kernels (collectives.cuh) run a tile through its phases one after the other: push, barrier,
// reduce / broadcast, barrier, copy out.  With a large message every CTA of every GPU is in the same phase
// at the same time, so NVLink is busy during the pushes and idle during the local copies, and every
// barrier exposes a release fence plus a flag flight.  Here a CTA works on three tiles at once, one per
// stage, and only ever waits for a signal that its peers sent one iteration earlier:
//
//   iteration k:   A(k)     push tile k                                    signal A(k)
//                  C(k-2D)  [wait B(k-2D)]  copy tile k-2D out              (three-stage kernels)
//                  B(k-D)   [wait A(k-D)]   reduce / broadcast tile k-D    signal B(k-D)
//
// D (Geometry::depth) is how many iterations lie between a tile's stages: a signal costs a release fence (the
// link has to drain what was queued before it) plus a flag flight, some 10 us on a busy link, and it is hidden
// when D iterations of other work take at least that long.  Tile k lives in staging buffer k mod R, R = 2D + 1
// buffers cut out of the CTA's 2 MiB of staging.  Why R are enough: buffer k mod R is written again by the
// peers' A(k+R); before that, in iteration k+R-1, they waited for B(k+R-1-2D) = B(k) of every rank.  What B
// writes (the gather area) is written again by the peers' B(k+R) after they waited for A(k+R), which a rank
// signals after its C(k) (iteration k+2D < k+R).  Two-stage kernels (ReduceScatter, AllGather) wait for
// B(k-R) before A(k).
//
// Signals are two monotonic counters per (CTA, peer): stream A in the ordinary pad row (the same words and
// the same epoch counter as block_barrier, of which a signal is one half), stream B in a second row.  They
// are issued by a warp of their own, so that the data warps never sit in a release fence (see PipeShared).
// A kernel starts and ends with a full barrier, because the plain kernels index the same staging bytes by
// halves: the first keeps the pushes away from a peer that is still copying out of the previous kernel's
// half, the last lets the next kernel write anywhere.  All waits are bounded like everywhere else.
//
// Status: opt-in (NANO_NCCL_PIPE_MIN_BYTES).  On two B200 every configuration tried was slower than the plain
// kernels: a signal is a release fence of about 5 us while the link is busy, the signalling warp issues two per
// iteration one after the other, and so an iteration costs about 10 us however small the tile is.  More
// signalling warps (fences in flight together, flags raised with a remote max) are the next step.
//
// The reference pipelines its ring the same way in spirit (up to four slices in flight per edge:
// src/kernels/ring_simple_kernel.cuh:1116-1438); this is that idea on one- and two-hop algorithms.
#pragma once

#include "kernels/collectives.cuh"

namespace nano_nccl::dev {

// Second flag row: word index of (block, rank) inside a rank's signal pads.  Below the fused-GEMM flags.
constexpr std::size_t kPipeFlagRowWords = 2048;
static_assert((kPipeFlagRowWords + kMaxBlocks * kPadWordsPerBlock) * 4 <= kGemmFlagOffsetBytes, "second flag row fits");

// Buffer of tile k: one of the 2 * depth + 1 buffers of this CTA's staging.
__device__ __forceinline__ std::size_t pipe_buf_offset(const Geometry& g, int k) {
    return static_cast<std::size_t>(blockIdx.x) * kBlockStageBytes +
           static_cast<std::size_t>(k % (2 * g.depth + 1)) * pipe_buf_bytes(g.depth);
}

// Roles inside a CTA: warps 0..14 (kPipeDataThreads) move data; warp 15 only signals.  A signal is a release
// store at system scope, i.e. a fence that waits until the CTA's earlier remote stores have been acknowledged
// over NVLink, which on a saturated link takes as long as draining everything queued before them.  If the data
// warps issued it themselves, every stage would end with that drain and nothing would overlap (measured: the
// pipeline was slower than the plain kernels).  So a data thread only arrives on a shared-memory mbarrier when
// a stage is done (release at CTA scope) and moves on; the signalling warp acquires the mbarrier phase, runs
// the fence and stores the flags.  The two release steps chain (CTA scope, then system scope), so a peer that
// acquires the flag sees the stage's data.
constexpr int kPipeDataThreads = kCollectiveThreads - 32;

struct PipeShared {
    std::uint64_t bar_a;                 // data threads arrive when stage A of a tile is issued
    std::uint64_t bar_b;                 // ... when stage B of a tile is done
    volatile std::uint32_t taken_a;      // phases of bar_a the signalling warp has consumed
    volatile std::uint32_t taken_b;
    volatile std::uint32_t failed;       // a bounded wait ran out somewhere in the CTA
    std::uint32_t giveup;                // wait_flag's cross-thread cancel word
    volatile std::uint32_t verdict;      // `failed` as thread 0 read it between two barriers: the same for every data thread
};

__device__ __forceinline__ void pipe_data_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kPipeDataThreads) : "memory"); }

// A data thread reports "stage done" for phase `index` of `bar`.  It first makes sure the signalling warp has
// consumed every earlier phase (an mbarrier tracks one pending phase), which it normally has long ago.
__device__ __forceinline__ void pipe_hand_over(const CommDev& c, PipeShared& sh, std::uint64_t* bar,
                                               volatile std::uint32_t* taken, std::uint32_t index) {
    if (*taken < index) {
        const unsigned long long start = global_timer_ns();
        while (*taken < index && sh.failed == 0u) {
            if (global_timer_ns() - start > c.timeout_ns) sh.failed = 1u;
        }
    }
    gemm::mbar_arrive(bar);
}

// Data threads: wait until every peer's flag word (row, this block) has reached `target`; uniform over the data warps.
__device__ __forceinline__ bool pipe_wait(const CommDev& c, PipeShared& sh, std::size_t row, std::uint32_t target, int phase) {
    const int peer = static_cast<int>(threadIdx.x);
    if (peer < c.nranks && peer != c.rank) {
        if (!wait_flag(c, c.pad[c.rank] + row + blockIdx.x * kPadWordsPerBlock + peer, target, peer, phase, &sh.giveup,
                       peer == (c.rank == 0 ? 1 : 0))) {
            sh.failed = 1u;
        }
    }
    // `failed` may be raised by the signalling warp at any moment, so the data warps must not each read it: one
    // thread reads it, and everybody uses that reading (a split decision would leave threads at different barriers).
    pipe_data_sync();
    if (threadIdx.x == 0) sh.verdict = sh.failed;
    pipe_data_sync();
    return sh.verdict == 0u;
}

// Signalling warp: acquire phase `index` of `bar` (bounded), then store `value` into the peers' flag words.
__device__ __forceinline__ bool pipe_signal_when_done(const CommDev& c, PipeShared& sh, std::uint64_t* bar,
                                                      volatile std::uint32_t* taken, std::uint32_t index, std::size_t row,
                                                      std::uint32_t value) {
    const unsigned long long start = global_timer_ns();
    unsigned spins = 0;
    while (!gemm::mbar_try_wait(bar, index & 1u)) {
        if ((++spins & 63u) == 0u) {
            if (sh.failed != 0u) return false;
            if (global_timer_ns() - start > 2 * c.timeout_ns) {
                sh.failed = 1u;
                return false;
            }
        }
    }
    const int lane = static_cast<int>(threadIdx.x) - kPipeDataThreads;
    if (lane == 0) *taken = index + 1u;
    if (lane < c.nranks && lane != c.rank) {
        st_release_sys(c.pad[lane] + row + blockIdx.x * kPadWordsPerBlock + c.rank, value);
    }
    return true;
}

// The schedule.  stage_a / stage_b / stage_c take the tile index and are run by the data threads (they must
// stride by kPipeDataThreads); kThree selects the three-stage form.
template <bool kThree, typename FA, typename FB, typename FC>
__device__ __forceinline__ void pipe_run(const CommDev& c, int tiles, int D, FA&& stage_a, FB&& stage_b, FC&& stage_c) {
    __shared__ PipeShared sh;
    std::uint32_t epoch = c.state[blockIdx.x].epoch;
    std::uint32_t epoch_b = c.state[blockIdx.x].epoch_b;
    const std::uint32_t seq = c.state[blockIdx.x].seq;
    if (threadIdx.x == 0) {
        gemm::mbar_init(&sh.bar_a, kPipeDataThreads);
        gemm::mbar_init(&sh.bar_b, kPipeDataThreads);
        sh.taken_a = 0u;
        sh.taken_b = 0u;
        sh.failed = 0u;
        sh.giveup = 0u;
        sh.verdict = 0u;
        gemm::fence_barrier_init();
    }
    bool ok = block_barrier(c, epoch, 1);  // also publishes the shared-memory set-up to every warp
    const std::uint32_t a0 = epoch, b0 = epoch_b;  // signal A(k) carries a0 + k + 1, signal B(k) carries b0 + k + 1
    const int R = 2 * D + 1;                                   // buffers
    const int last = tiles - 1 + (kThree ? 2 * D : D);         // last iteration with work
    if (ok && threadIdx.x >= kPipeDataThreads) {
        // ---- signalling warp: the data warps' hand-overs in their program order
        for (int k = 0; k <= last; ++k) {
            if (k < tiles && !pipe_signal_when_done(c, sh, &sh.bar_a, &sh.taken_a, static_cast<std::uint32_t>(k), 0,
                                                    a0 + static_cast<std::uint32_t>(k) + 1u)) break;
            if (k >= D && k - D < tiles &&
                !pipe_signal_when_done(c, sh, &sh.bar_b, &sh.taken_b, static_cast<std::uint32_t>(k - D), kPipeFlagRowWords,
                                       b0 + static_cast<std::uint32_t>(k - D) + 1u)) break;
        }
    } else if (ok) {
        // ---- data warps
        for (int k = 0; k <= last; ++k) {
            if (k < tiles) {
                // two-stage kernels: the buffer is free once every peer has consumed the tile that used it last
                if (!kThree && k >= R && !pipe_wait(c, sh, kPipeFlagRowWords, b0 + static_cast<std::uint32_t>(k - R) + 1u, 3)) break;
                stage_a(k);
                pipe_hand_over(c, sh, &sh.bar_a, &sh.taken_a, static_cast<std::uint32_t>(k));
            }
            if (kThree && k >= 2 * D && k - 2 * D < tiles) {
                if (!pipe_wait(c, sh, kPipeFlagRowWords, b0 + static_cast<std::uint32_t>(k - 2 * D) + 1u, 4)) break;
                stage_c(k - 2 * D);
            }
            if (k >= D && k - D < tiles) {
                if (!pipe_wait(c, sh, 0, a0 + static_cast<std::uint32_t>(k - D) + 1u, 3)) break;
                stage_b(k - D);
                pipe_hand_over(c, sh, &sh.bar_b, &sh.taken_b, static_cast<std::uint32_t>(k - D));
            }
        }
    }
    __syncthreads();
    ok = ok && sh.failed == 0u;
    if (ok) {
        epoch = a0 + static_cast<std::uint32_t>(tiles);
        epoch_b = b0 + static_cast<std::uint32_t>(tiles);
        block_barrier(c, epoch, 2);
    }
    if (threadIdx.x == 0) {
        c.state[blockIdx.x].epoch = epoch;
        c.state[blockIdx.x].epoch_b = epoch_b;
        c.state[blockIdx.x].seq = seq;
    }
}

// Copies `nvec` 16-byte vectors with kPipeBatch loads in flight per data thread.  LoadFn(v) -> Vec16, StoreFn(v, x).
// Four per thread (1920 per CTA, 30 KiB) cover the bandwidth-delay product of a CTA's share of NVLink several
// times over and leave the three inlined stages enough registers under the 128-register cap of a 512-thread CTA.
constexpr int kPipeBatch = 4;
template <typename LoadFn, typename StoreFn>
__device__ __forceinline__ void batched_copy(std::size_t nvec, LoadFn&& load, StoreFn&& store) {
    for (std::size_t v0 = threadIdx.x; v0 < nvec; v0 += kPipeBatch * kPipeDataThreads) {
        Vec16 x[kPipeBatch];
#pragma unroll
        for (int k = 0; k < kPipeBatch; ++k) {
            const std::size_t v = v0 + k * kPipeDataThreads;
            if (v < nvec) x[k] = load(v);
        }
#pragma unroll
        for (int k = 0; k < kPipeBatch; ++k) {
            const std::size_t v = v0 + k * kPipeDataThreads;
            if (v < nvec) store(v, x[k]);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Two-shot AllReduce, pipelined.  A buffer is split into a scatter half and a gather half of N slots each;
// g.slot_bytes = bytes of one rank's sub-slice of a tile.
template <typename T, RedOp Op, bool kMc>
__device__ __forceinline__ void
ar_twoshot_pipe_body(const CommDev& c, const T* src, T* dst, std::size_t count, const Geometry g) {
    constexpr int kE = ElemsPerVec<T>::value;
    const std::size_t kGatherOff = pipe_buf_bytes(g.depth) / 2;
    const float inv = 1.0f / static_cast<float>(c.nranks);
    const int N = c.nranks;
    auto tile = [&](int k, std::size_t* t0, std::size_t* n) { tile_range(count, g, k, t0, n); };
    auto stage_a = [&](int k) {  // sub-slice j of my tile goes to rank j
        std::size_t t0, n;
        tile(k, &t0, &n);
        if (!tile_fits(c, max_split_bytes<T>(n, N), g.slot_bytes, N, kGatherOff)) return;
        const std::size_t off = pipe_buf_offset(g, k);
        const T* s = src + t0;
        const bool s_al = aligned16(s);
        for (int i = 1; i < N; ++i) {
            const int j = (c.rank + i) % N;
            const std::size_t b = split_begin(n, N, j, kE), e = split_begin(n, N, j + 1, kE);
            const std::size_t len = e - b;
            char* out = c.stage[j] + off + c.rank * g.slot_bytes;
            batched_copy((len + kE - 1) / kE, [&](std::size_t v) { return load_guarded(s + b, v * kE, len, s_al); },
                         [&](std::size_t v, const Vec16& x) { st_vec(out + v * 16, x); });
        }
    };
    auto stage_b = [&](int k) {  // reduce my sub-slice in rank order, write it to my output and to everyone's gather half
        std::size_t t0, n;
        tile(k, &t0, &n);
        if (!tile_fits(c, max_split_bytes<T>(n, N), g.slot_bytes, N, kGatherOff)) return;
        const std::size_t off = pipe_buf_offset(g, k);
        const T* s = src + t0;
        T* d = dst + t0;
        const bool s_al = aligned16(s), d_al = aligned16(d);
        const std::size_t b = split_begin(n, N, c.rank, kE), e = split_begin(n, N, c.rank + 1, kE);
        const std::size_t len = e - b, nvec = (len + kE - 1) / kE;
        const char* in = c.stage[c.rank] + off;
        const std::size_t go = off + kGatherOff + c.rank * g.slot_bytes;
        for (std::size_t v = threadIdx.x; v < nvec; v += kPipeDataThreads) {
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
    };
    auto stage_c = [&](int k) {  // the other owners' results leave my gather half
        std::size_t t0, n;
        tile(k, &t0, &n);
        const std::size_t off = pipe_buf_offset(g, k);
        T* d = dst + t0;
        const bool d_al = aligned16(d);
        for (int i = 1; i < N; ++i) {
            const int j = (c.rank + i) % N;
            const std::size_t b = split_begin(n, N, j, kE), e = split_begin(n, N, j + 1, kE);
            const std::size_t len = e - b;
            const char* in = c.stage[c.rank] + off + kGatherOff + j * g.slot_bytes;
            batched_copy((len + kE - 1) / kE, [&](std::size_t v) { return ld_vec_volatile(in + v * 16); },
                         [&](std::size_t v, const Vec16& x) { store_guarded(d + b, v * kE, len, d_al, x); });
        }
    };
    pipe_run<true>(c, g.iters, g.depth, stage_a, stage_b, stage_c);
}

// ------------------------------------------------------------------------------------------------
// AllReduce through the switch, pipelined: A copies the tile into the multicast-bound buffer, B reduces the
// owned slice in the switch and writes the result into every rank's buffer, C copies the rest out.
template <typename T, RedOp Op>
__device__ __forceinline__ void
ar_nvls_pipe_body(const CommDev& c, const T* src, T* dst, std::size_t count, const Geometry g) {
    static_assert(Op == RedOp::Sum || Op == RedOp::Avg, "the switch only adds");
    constexpr int kE = ElemsPerVec<T>::value;
    const float inv = 1.0f / static_cast<float>(c.nranks);
    const int N = c.nranks;
    auto stage_a = [&](int k) {
        std::size_t t0, n;
        tile_range(count, g, k, &t0, &n);
        const std::size_t nvec = (n + kE - 1) / kE;
        if (!tile_fits(c, nvec * 16, pipe_buf_bytes(g.depth), 1, pipe_buf_bytes(g.depth))) return;
        char* mine = c.stage[c.rank] + pipe_buf_offset(g, k);
        const T* s = src + t0;
        const bool s_al = aligned16(s);
        batched_copy(nvec, [&](std::size_t v) { return load_guarded(s, v * kE, n, s_al); },
                     [&](std::size_t v, const Vec16& x) { st_vec(mine + v * 16, x); });
    };
    auto stage_b = [&](int k) {
        std::size_t t0, n;
        tile_range(count, g, k, &t0, &n);
        const std::size_t nvec = (n + kE - 1) / kE;
        if (!tile_fits(c, nvec * 16, pipe_buf_bytes(g.depth), 1, pipe_buf_bytes(g.depth))) return;
        const std::size_t off = pipe_buf_offset(g, k);
        T* d = dst + t0;
        const bool d_al = aligned16(d);
        const std::size_t b = split_begin(n, N, c.rank, kE), e = split_begin(n, N, c.rank + 1, kE);
        const std::size_t vb = (b + kE - 1) / kE, ve = (e + kE - 1) / kE;  // b == n when the slice is empty
        batched_copy(ve - vb, [&](std::size_t v) { return multimem_ld_reduce_add<T>(c.stage_mc + off + (vb + v) * 16); },
                     [&](std::size_t v, Vec16 x) {
                         if constexpr (Op == RedOp::Avg) {
                             Acc<T> a = unpack<T>(x);
                             finish<Op, T>(a, inv);
                             x = pack<T>(a);
                         }
                         multimem_st(c.stage_mc + off + (vb + v) * 16, x);
                         store_guarded(d, (vb + v) * kE, n, d_al, x);
                     });
    };
    auto stage_c = [&](int k) {
        std::size_t t0, n;
        tile_range(count, g, k, &t0, &n);
        const std::size_t nvec = (n + kE - 1) / kE;
        const char* mine = c.stage[c.rank] + pipe_buf_offset(g, k);
        T* d = dst + t0;
        const bool d_al = aligned16(d);
        const std::size_t b = split_begin(n, N, c.rank, kE), e = split_begin(n, N, c.rank + 1, kE);
        const std::size_t vb = (b + kE - 1) / kE, ve = (e + kE - 1) / kE;
        // everything but my own slice: [0, vb) and [ve, nvec)
        const std::size_t rest = nvec - (ve - vb);
        batched_copy(rest, [&](std::size_t v) { return ld_vec_volatile(mine + (v < vb ? v : v + (ve - vb)) * 16); },
                     [&](std::size_t v, const Vec16& x) { store_guarded(d, (v < vb ? v : v + (ve - vb)) * kE, n, d_al, x); });
    };
    pipe_run<true>(c, g.iters, g.depth, stage_a, stage_b, stage_c);
}

// ------------------------------------------------------------------------------------------------
// ReduceScatter, pipelined (two stages).  `count` = recv_count; g.slot_bytes = bytes of a tile.
template <typename T, RedOp Op>
__device__ __forceinline__ void
rs_pipe_body(const CommDev& c, const T* src, T* dst, std::size_t count, const Geometry g) {
    constexpr int kE = ElemsPerVec<T>::value;
    const float inv = 1.0f / static_cast<float>(c.nranks);
    const int N = c.nranks;
    auto stage_a = [&](int k) {
        std::size_t t0, n;
        tile_range(count, g, k, &t0, &n);
        const std::size_t nvec = (n + kE - 1) / kE;
        if (!tile_fits(c, nvec * 16, g.slot_bytes, N, pipe_buf_bytes(g.depth))) return;
        const std::size_t off = pipe_buf_offset(g, k);
        for (int i = 1; i < N; ++i) {
            const int j = (c.rank + i) % N;
            const T* s = src + static_cast<std::size_t>(j) * count + t0;
            const bool s_al = aligned16(s);
            char* out = c.stage[j] + off + c.rank * g.slot_bytes;
            batched_copy(nvec, [&](std::size_t v) { return load_guarded(s, v * kE, n, s_al); },
                         [&](std::size_t v, const Vec16& x) { st_vec(out + v * 16, x); });
        }
    };
    auto stage_b = [&](int k) {
        std::size_t t0, n;
        tile_range(count, g, k, &t0, &n);
        const std::size_t nvec = (n + kE - 1) / kE;
        if (!tile_fits(c, nvec * 16, g.slot_bytes, N, pipe_buf_bytes(g.depth))) return;
        const T* own = src + static_cast<std::size_t>(c.rank) * count + t0;
        const bool own_al = aligned16(own);
        T* d = dst + t0;
        const bool d_al = aligned16(d);
        const char* in = c.stage[c.rank] + pipe_buf_offset(g, k);
        for (std::size_t v = threadIdx.x; v < nvec; v += kPipeDataThreads) {
            Acc<T> acc;
            for (int r = 0; r < N; ++r) {
                const Vec16 x = (r == c.rank) ? load_guarded(own, v * kE, n, own_al)
                                              : ld_vec_volatile(in + r * g.slot_bytes + v * 16);
                if (r == 0) acc = unpack<T>(x); else combine<Op, T>(acc, unpack<T>(x));
            }
            finish<Op, T>(acc, inv);
            store_guarded(d, v * kE, n, d_al, pack<T>(acc));
        }
    };
    pipe_run<false>(c, g.iters, g.depth, stage_a, stage_b, [](int) {});
}

// ------------------------------------------------------------------------------------------------
// AllGather, pipelined (two stages).  `count` = send_count; g.slot_bytes = bytes of a tile.
template <typename T, bool kMc>
__device__ __forceinline__ void
ag_pipe_body(const CommDev& c, const T* src, T* dst, std::size_t count, const Geometry g) {
    constexpr int kE = ElemsPerVec<T>::value;
    const int N = c.nranks;
    auto stage_a = [&](int k) {
        std::size_t t0, n;
        tile_range(count, g, k, &t0, &n);
        const std::size_t nvec = (n + kE - 1) / kE;
        if (!tile_fits(c, nvec * 16, g.slot_bytes, N, pipe_buf_bytes(g.depth))) return;
        const std::size_t off = pipe_buf_offset(g, k) + c.rank * g.slot_bytes;
        const T* s = src + t0;
        const bool s_al = aligned16(s);
        T* own = dst + static_cast<std::size_t>(c.rank) * count + t0;
        const bool own_al = aligned16(own);
        batched_copy(nvec, [&](std::size_t v) { return load_guarded(s, v * kE, n, s_al); },
                     [&](std::size_t v, const Vec16& x) {
                         store_guarded(own, v * kE, n, own_al, x);
                         if constexpr (kMc) {
                             multimem_st(c.stage_mc + off + v * 16, x);
                         } else {
                             for (int i = 1; i < N; ++i) st_vec(c.stage[(c.rank + i) % N] + off + v * 16, x);
                         }
                     });
    };
    auto stage_b = [&](int k) {
        std::size_t t0, n;
        tile_range(count, g, k, &t0, &n);
        const std::size_t nvec = (n + kE - 1) / kE;
        if (!tile_fits(c, nvec * 16, g.slot_bytes, N, pipe_buf_bytes(g.depth))) return;
        const std::size_t off = pipe_buf_offset(g, k);
        for (int i = 1; i < N; ++i) {
            const int j = (c.rank + i) % N;
            T* d = dst + static_cast<std::size_t>(j) * count + t0;
            const bool d_al = aligned16(d);
            const char* in = c.stage[c.rank] + off + j * g.slot_bytes;
            batched_copy(nvec, [&](std::size_t v) { return ld_vec_volatile(in + v * 16); },
                         [&](std::size_t v, const Vec16& x) { store_guarded(d, v * kE, n, d_al, x); });
        }
    };
    pipe_run<false>(c, g.iters, g.depth, stage_a, stage_b, [](int) {});
}

// ------------------------------------------------------------------------------------------------
template <typename T, RedOp Op, bool kMc>
NANO_KERNEL ar_twoshot_pipe_kernel(CommDev c, const T* src, T* dst, std::size_t count, const Geometry g) {
    ar_twoshot_pipe_body<T, Op, kMc>(c, src, dst, count, g);
}
template <typename T, RedOp Op>
NANO_KERNEL ar_twoshot_pipe_emu_kernel(const EmuRanks* e, std::size_t count, const Geometry g) {
    const int r = blockIdx.y;
    ar_twoshot_pipe_body<T, Op, false>(e->ctx[r], static_cast<const T*>(e->src[r]), static_cast<T*>(e->dst[r]), count, g);
}
template <typename T, RedOp Op>
NANO_KERNEL ar_nvls_pipe_kernel(CommDev c, const T* src, T* dst, std::size_t count, const Geometry g) {
    ar_nvls_pipe_body<T, Op>(c, src, dst, count, g);
}
template <typename T, RedOp Op>
NANO_KERNEL rs_pipe_kernel(CommDev c, const T* src, T* dst, std::size_t count, const Geometry g) {
    rs_pipe_body<T, Op>(c, src, dst, count, g);
}
template <typename T, RedOp Op>
NANO_KERNEL rs_pipe_emu_kernel(const EmuRanks* e, std::size_t count, const Geometry g) {
    const int r = blockIdx.y;
    rs_pipe_body<T, Op>(e->ctx[r], static_cast<const T*>(e->src[r]), static_cast<T*>(e->dst[r]), count, g);
}
template <typename T, bool kMc>
NANO_KERNEL ag_pipe_kernel(CommDev c, const T* src, T* dst, std::size_t count, const Geometry g) {
    ag_pipe_body<T, kMc>(c, src, dst, count, g);
}
template <typename T>
NANO_KERNEL ag_pipe_emu_kernel(const EmuRanks* e, std::size_t count, const Geometry g) {
    const int r = blockIdx.y;
    ag_pipe_body<T, false>(e->ctx[r], static_cast<const T*>(e->src[r]), static_cast<T*>(e->dst[r]), count, g);
}

}  // namespace nano_nccl::dev
