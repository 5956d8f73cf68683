// Persistent, warp-specialised BF16 GEMM for sm_100a: C[M,N] = A[M,K] * B[N,K]^T (+ bias), fp32
// accumulation in TMEM.  The same kernel body carries the two fused tensor-parallel variants:
//
//   Mode::Plain    epilogue stores the tile to local memory.
//   Mode::GemmRs   row-parallel GEMM -> ReduceScatter over rows: the tile grid is walked owner by
//                  owner, starting with the next rank's rows and ending with this rank's own rows.
//                  The epilogue of a foreign tile stores the bf16 partial straight into the owner
//                  GPU's staging slot over NVLink and then raises that tile's flag there; the
//                  epilogue of an own tile waits for the N-1 flags, adds the N-1 staged partials
//                  to its fp32 accumulator and writes the final rows.  Transfer of tile i overlaps
//                  the MMA of tile i+1 (double-buffered TMEM accumulators).
//   Mode::AgGemm   AllGather -> column-parallel GEMM: a few CTAs push this rank's activation shard
//                  into every GPU's gathered buffer (one multimem.st per 16 bytes, or P2P stores)
//                  block by block, and raise flags per 128-row block; the GEMM CTAs start with the local shard
//                  and gate the TMA loads of each remote row block on its flag.  TMA only ever
//                  reads this GPU's own memory, without multicast.
//
// Roles per CTA (192 threads): warp 0 = TMA producer (one elected lane), warp 1 = MMA issuer (one
// elected lane; also owns the TMEM allocation), warps 2..5 = epilogue (TMEM lane quadrant =
// warp_id % 4).  Tile 128 x 256 x 64, 4 smem stages (48 KB each), 2 TMEM accumulators of 256
// columns.  Every wait is bounded; on expiry the CTA records an error code, stops issuing work
// and leaves through the common teardown, which frees TMEM.
//
// No counterpart in the reference (it has no GEMM); these are the new fused tensor-parallel
// kernels the framework adds on top of the collective library.
#pragma once

#include "gemm/tcgen05.cuh"
#include "kernels/bulk_pipe.cuh"
#include "kernels/prims.cuh"

namespace nano_nccl::gemm {

constexpr int kBM = 128, kBN = 256, kBK = 64;
constexpr int kStages = 4;
constexpr int kAccStages = 2;
constexpr int kTmemCols = 512;
constexpr int kGemmThreads = 224;      // warp 0 TMA, 1 MMA, 2..5 epilogue, 6 publishes the tile flags of GemmRs
constexpr int kEpilogueThreads = 128;
constexpr int kPublisherWarp = 6;
constexpr std::uint32_t kStageBytesA = kBM * kBK * 2;
constexpr std::uint32_t kStageBytesB = kBN * kBK * 2;
constexpr std::uint32_t kStageBytes = kStageBytesA + kStageBytesB;
constexpr int kEpiCols = 128;                                   // columns staged per pass
constexpr std::uint32_t kEpiRowBytes = kEpiCols * 2;            // 256 B of bf16 per row
constexpr std::uint32_t kEpiWarpBytes = 32 * kEpiRowBytes;      // one warp stages its 32 rows
constexpr std::uint32_t kEpiBytes = 4 * kEpiWarpBytes;          // 32 KB
constexpr std::uint32_t kTmaBoxBytes = 32 * 128;                // one 64-column x 32-row box of bf16
constexpr int kMaxPushParts = 32;                               // AgGemm: most push units a 128-row block is cut into
constexpr std::size_t kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget of one CTA");
static_assert((2 * kStages + 2 * kAccStages + 1) * 8 + 12 <= 256, "barrier area");

// GemmRsTma is GemmRs with the remote part of the epilogue done by the TMA unit: a foreign tile is
// staged in shared memory in the 128-byte-swizzle layout and written into the owner's staging with
// tensor stores (two 64-column boxes per warp and pass), so the epilogue warps issue two
// instructions instead of sixteen remote vector stores per pass and never wait for NVLink.
enum class Mode { Plain, GemmRs, AgGemm, GemmRsTma };

template <Mode kMode>
inline constexpr bool kIsRs = kMode == Mode::GemmRs || kMode == Mode::GemmRsTma;

// Tensor maps of every rank's GemmRs staging ([nranks * rows_per_rank][N] bf16, box 64 x 32,
// 128-byte swizzle); only GemmRsTma reads them.
struct PeerMaps {
    CUtensorMap m[kMaxRanks];
};

enum GemmError : int {
    kGemmOk = 0,
    kGemmWaitProducer = 1,   // smem stage never freed
    kGemmWaitMma = 2,        // TMA data never arrived / accumulator never freed
    kGemmWaitEpilogue = 3,   // accumulator never completed
    kGemmWaitPeer = 4,       // a peer's flag never arrived
};

struct FusedArgs {
    int rank = 0;
    int nranks = 1;
    std::uint32_t epoch = 1;                       // flag value of this call
    // GemmRs: staging[r] = rank r's receive area, laid out [src_rank][rows_per_rank][N] bf16;
    // flags[r] = rank r's flag array [src_rank][tiles_per_owner].
    __nv_bfloat16* staging[kMaxRanks] = {};
    std::uint32_t* flags[kMaxRanks] = {};
    // AgGemm: gathered[r] = rank r's gathered activation buffer [M][K]; gathered_mc = multicast
    // alias (nullptr: P2P stores); shard = this rank's [M / nranks][K] input.
    __nv_bfloat16* gathered[kMaxRanks] = {};
    __nv_bfloat16* gathered_mc = nullptr;
    std::uint32_t* flags_mc = nullptr;
    const __nv_bfloat16* shard = nullptr;
    int push_ctas = 0;                             // AgGemm: CTAs [0, push_ctas) only move data
    int push_tma = 0;                              // AgGemm: pushers use TMA bulk copies (unicast to every peer)
    // AgGemm: a 128-row block is pushed as push_parts units (a power of two <= kMaxPushParts) by different
    // pusher CTAs, so that the pushers finish block b before they start block b + 1 and the GEMM can follow
    // the blocks as they arrive instead of waiting for the whole shard.
    int push_parts = 2;
    // Diagnostic time line (null: off).  kTraceSlots words per CTA and role: role 0 = the epilogue's first
    // thread, role 1 = the TMA producer (AgGemm) or the flag publisher (GemmRs).  A word is
    // (tag << 60) | %globaltimer: tag 0 kernel entry, 1 accumulator complete, 2 the peers' partials have
    // arrived (own tiles), 3 accumulator handed back, 7 all four warps have issued a foreign tile's stores,
    // 4 that tile's flag published, 5 / 6 producer starts / ends waiting for a remote row block.
    unsigned long long* trace = nullptr;
    unsigned long long timeout_ns = 0;
};

struct GemmArgs {
    int M = 0, N = 0, K = 0;
    __nv_bfloat16* C = nullptr;      // Plain / AgGemm: [M][N]; GemmRs: [M / nranks][N]
    int ldc = 0;
    const __nv_bfloat16* bias = nullptr;
    int* error = nullptr;            // first error code, 0 when fine
    // Columns per tile: kBN, or a smaller multiple of 32 (of 64 with tensor stores) chosen by the host so
    // that the tile count fills whole waves of CTAs; shared memory and TMEM are laid out for kBN either way.
    int bn = kBN;
    // Plain mode: linear tile indices >= tail_first (the last, partly filled round of the persistent walk) are cut
    // into bn / tail_bn column pieces of tail_bn columns each, loaded through a tensor map of B whose box is that
    // narrow; tail_bn == 0: no split.
    int tail_first = 0;
    int tail_bn = 0;
};

constexpr int kTraceSlots = 128;

__device__ __forceinline__ void trace_stamp(const FusedArgs& f, int role, int* slot, unsigned long long tag) {
    if (f.trace != nullptr && *slot < kTraceSlots) {
        f.trace[(static_cast<std::size_t>(blockIdx.x) * 2 + role) * kTraceSlots + (*slot)++] =
            (tag << 60) | (dev::global_timer_ns() & ((1ull << 60) - 1));
    }
}

__device__ __forceinline__ void gemm_fail(const GemmArgs& g, int code, volatile int* abort_flag) {
    atomicCAS(g.error, 0, code);
    *abort_flag = 1;
}

// Maps a linear tile index of this CTA's walk to tile coordinates.
// Plain: row-major over (m_tiles x n_tiles), n fastest so that CTAs running together share A rows
// and the 16 column tiles of B stay in L2.
// GemmRs: owner-major.  step s in [0, nranks): owner = (rank + 1 + s) % nranks; inside an owner
// the same (m,n) order.  AgGemm: shard-major, starting with the local shard.
template <Mode kMode>
__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, const FusedArgs& f, int* tm,
                                            int* tn, int* owner) {
    if constexpr (kMode == Mode::Plain) {
        *tm = t / n_tiles;
        *tn = t % n_tiles;
        *owner = 0;
    } else if constexpr (kIsRs<kMode>) {
        const int m_per = m_tiles / f.nranks;             // row tiles per rank block
        const int per_owner = m_per * n_tiles;
        const int step = t / per_owner;
        const int in = t % per_owner;
        const int who = (f.rank + 1 + step) % f.nranks;
        *owner = who;
        *tm = who * m_per + in / n_tiles;
        *tn = in % n_tiles;
    } else {
        // AgGemm: the local shard first; then remote rows in the order they arrive: every rank
        // pushes its 128-row blocks in ascending order, so block b of all sources comes before
        // block b+1 of any.
        const int m_per = m_tiles / f.nranks;
        const int per_owner = m_per * n_tiles;
        if (t < per_owner) {
            *owner = f.rank;
            *tm = f.rank * m_per + t / n_tiles;
            *tn = t % n_tiles;
        } else {
            const int u = t - per_owner;
            const int per_block = (f.nranks - 1) * n_tiles;
            const int b = u / per_block;
            const int rem = u % per_block;
            const int who = (f.rank + 1 + rem / n_tiles) % f.nranks;
            *owner = who;
            *tm = who * m_per + b;
            *tn = rem % n_tiles;
        }
    }
}

// One item of a CTA's walk: an output tile, or in Plain mode a column piece of a tile of the last round.
struct TileWork {
    int tm, tn, owner;
    int col0;   // first output column
    int bn;     // columns computed
    bool tail;  // a piece: B comes through the narrow tensor map
};

template <Mode kMode>
__device__ __forceinline__ TileWork tile_work(int t, int m_tiles, int n_tiles, const GemmArgs& g, const FusedArgs& f) {
    TileWork w;
    w.bn = g.bn;
    w.tail = false;
    int lin = t, col_off = 0;
    if constexpr (kMode == Mode::Plain) {
        if (g.tail_bn > 0 && t >= g.tail_first) {
            const int pieces = g.bn / g.tail_bn;
            const int p = t - g.tail_first;
            lin = g.tail_first + p / pieces;
            col_off = (p % pieces) * g.tail_bn;
            w.bn = g.tail_bn;
            w.tail = true;
        }
    }
    tile_coords<kMode>(lin, m_tiles, n_tiles, f, &w.tm, &w.tn, &w.owner);
    w.col0 = w.tn * g.bn + col_off;
    return w;
}

template <Mode kMode>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_aux, GemmArgs g, FusedArgs f,
                 const __grid_constant__ PeerMaps peer_maps) {
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle atom (8 rows x 128 B)
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<std::uintptr_t>(smem_raw) + 1023) & ~std::uintptr_t{1023});
    unsigned char* smem_a = smem;
    unsigned char* smem_b = smem + kStages * kStageBytesA;
    unsigned char* smem_epi = smem + kStages * kStageBytes;
    std::uint64_t* bars = reinterpret_cast<std::uint64_t*>(smem + kStages * kStageBytes + kEpiBytes);
    std::uint64_t* full_bar = bars;                          // [kStages]
    std::uint64_t* empty_bar = bars + kStages;               // [kStages]
    std::uint64_t* acc_full = bars + 2 * kStages;            // [kAccStages]
    std::uint64_t* acc_empty = bars + 2 * kStages + kAccStages;  // [kAccStages]
    std::uint64_t* epi_bar = bars + 2 * kStages + 2 * kAccStages;  // epilogue warps -> flag publisher
    std::uint32_t* tmem_slot = reinterpret_cast<std::uint32_t*>(bars + 2 * kStages + 2 * kAccStages + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // phases of epi_bar the publisher has seen complete; an epilogue warp arrives for its j-th foreign tile
    // only once this is >= j, so an arrival can never count toward an earlier tile's phase
    volatile std::uint32_t* epi_seen = reinterpret_cast<volatile std::uint32_t*>(tmem_slot + 2);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int m_tiles = (g.M + kBM - 1) / kBM;
    const int n_tiles = (g.N + g.bn - 1) / g.bn;
    const int k_blocks = (g.K + kBK - 1) / kBK;
    // tmap_aux: AgGemm: this rank's un-gathered shard; Plain: B with the narrow box of the tail pieces
    int total_tiles = m_tiles * n_tiles;
    if constexpr (kMode == Mode::Plain) {
        if (g.tail_bn > 0) total_tiles = g.tail_first + (total_tiles - g.tail_first) * (g.bn / g.tail_bn);
    }

    int first_cta = 0, num_ctas = static_cast<int>(gridDim.x);
    if constexpr (kMode == Mode::AgGemm) {
        first_cta = f.push_ctas;
        num_ctas -= f.push_ctas;
    }

    // ---------------------------------------------------------------- AgGemm: data-moving CTAs
    if constexpr (kMode == Mode::AgGemm) {
        if (static_cast<int>(blockIdx.x) < f.push_ctas) {
            // Push this rank's shard, 128-row block by block, into every rank's gathered buffer at
            // rows [rank * rows_per, ...), then raise flag[rank][block] everywhere.
            const int rows_per = g.M / f.nranks;
            const int units = (rows_per / kBM) * f.push_parts;
            const int unit_rows = kBM / f.push_parts;
            const std::size_t vec_per_unit = static_cast<std::size_t>(unit_rows) * g.K * 2 / 16;
            if (f.push_tma != 0) {
                // One thread moves each unit through a ring of shared-memory stages with bulk copies: global ->
                // shared once, shared -> every peer's gathered buffer.  The SM issues a handful of instructions
                // per 16 KB; the TMA unit does the NVLink writes.
                static_assert(dev::kPipeSmemBytes <= kStages * kStageBytes, "the pipe lives in the operand stages");
                dev::BulkPipe pipe;
                dev::pipe_init(pipe, smem);
                const std::size_t unit_bytes = static_cast<std::size_t>(unit_rows) * g.K * 2;
                for (int u = blockIdx.x; u < units; u += f.push_ctas) {
                    if (threadIdx.x == 0) {
                        const char* src = reinterpret_cast<const char*>(f.shard + static_cast<std::size_t>(u) * unit_rows * g.K);
                        const std::size_t dst_off =
                            (static_cast<std::size_t>(f.rank) * rows_per + static_cast<std::size_t>(u) * unit_rows) * g.K * 2;
                        char* targets[kMaxRanks];
                        int nt = 0;
                        for (int i = 1; i < f.nranks; ++i) {
                            targets[nt++] = reinterpret_cast<char*>(f.gathered[(f.rank + i) % f.nranks]) + dst_off;
                        }
                        if (!dev::pipe_push(pipe, src, targets, nt, unit_bytes)) atomicCAS(g.error, 0, kGemmWaitProducer);
                        __threadfence_system();
                    }
                    __syncthreads();
                    if (threadIdx.x < static_cast<unsigned>(f.nranks) && static_cast<int>(threadIdx.x) != f.rank) {
                        dev::st_release_sys(f.flags[threadIdx.x] + f.rank * units + u, f.epoch);
                    }
                }
                return;
            }
            for (int u = blockIdx.x; u < units; u += f.push_ctas) {
                const char* src = reinterpret_cast<const char*>(f.shard + static_cast<std::size_t>(u) * unit_rows * g.K);
                const std::size_t dst_off = (static_cast<std::size_t>(f.rank) * rows_per + static_cast<std::size_t>(u) * unit_rows) * g.K * 2;
                constexpr int kPushBatch = 8;  // 16-byte loads each thread keeps in flight
                for (std::size_t v0 = threadIdx.x; v0 < vec_per_unit; v0 += kPushBatch * blockDim.x) {
                    dev::Vec16 x[kPushBatch];
#pragma unroll
                    for (int k = 0; k < kPushBatch; ++k) {
                        const std::size_t v = v0 + k * blockDim.x;
                        if (v < vec_per_unit) x[k] = dev::ld_vec_stream(src + v * 16);
                    }
#pragma unroll
                    for (int k = 0; k < kPushBatch; ++k) {
                        const std::size_t v = v0 + k * blockDim.x;
                        if (v < vec_per_unit) {
                            if (f.gathered_mc != nullptr) {
                                dev::multimem_st(reinterpret_cast<char*>(f.gathered_mc) + dst_off + v * 16, x[k]);
                            } else {
                                for (int i = 1; i < f.nranks; ++i) {
                                    const int p = (f.rank + i) % f.nranks;
                                    dev::st_vec(reinterpret_cast<char*>(f.gathered[p]) + dst_off + v * 16, x[k]);
                                }
                            }
                        }
                    }
                }
                __syncthreads();
                if (threadIdx.x < static_cast<unsigned>(f.nranks) && static_cast<int>(threadIdx.x) != f.rank) {
                    // release: the unit's stores (ordered by the barrier above) precede the flag
                    dev::st_release_sys(f.flags[threadIdx.x] + f.rank * units + u, f.epoch);
                }
            }
            return;
        }
    }

    // ---------------------------------------------------------------- setup
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < kAccStages; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], kEpilogueThreads / 32);
        }
        mbar_init(epi_bar, kEpilogueThreads / 32);
        *abort_flag = 0;
        *epi_seen = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
    }
    if (warp == 1) tmem_alloc<kTmemCols>(tmem_slot);
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const std::uint32_t tmem_base = *tmem_slot;
    const int cta = static_cast<int>(blockIdx.x) - first_cta;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (elect_one()) {
            int stage = 0;
            int producer_slot = 0;
            std::uint32_t phase = 0;
            for (int t = cta; t < total_tiles && *abort_flag == 0; t += num_ctas) {
                const TileWork w = tile_work<kMode>(t, m_tiles, n_tiles, g, f);
                const int tm = w.tm, owner = w.owner;
                if constexpr (kMode == Mode::AgGemm) {
                    if (owner != f.rank) {
                        // rows of a remote shard: wait until its pusher raised this block's flag
                        const int blocks = g.M / f.nranks / kBM;
                        const int b = tm - owner * blocks;
                        const std::uint32_t* flag = f.flags[f.rank] + owner * blocks * f.push_parts + b * f.push_parts;
                        const unsigned long long start = dev::global_timer_ns();
                        unsigned spins = 0;
                        bool ok = true;
                        trace_stamp(f, 1, &producer_slot, 5);
                        for (int part = 0; part < f.push_parts && ok; ++part) {
                            while (static_cast<std::int32_t>(dev::ld_acquire_sys(flag + part) - f.epoch) < 0) {
                                if ((++spins & 63u) == 0u && dev::global_timer_ns() - start > f.timeout_ns) {
                                    ok = false;
                                    break;
                                }
                            }
                        }
                        if (!ok) {
                            gemm_fail(g, kGemmWaitPeer, abort_flag);
                            break;
                        }
                        trace_stamp(f, 1, &producer_slot, 6);
                        // the rows were written by another GPU through the generic proxy; TMA
                        // reads through the async proxy
                        asm volatile("fence.proxy.async;" ::: "memory");
                    }
                }
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u)) {
                        gemm_fail(g, kGemmWaitProducer, abort_flag);
                        break;
                    }
                    mbar_arrive_expect_tx(&full_bar[stage], kStageBytesA + static_cast<std::uint32_t>(w.bn) * kBK * 2);
                    if (kMode == Mode::AgGemm && owner == f.rank) {
                        // own rows come straight from the un-gathered shard
                        tma_load_2d(smem_a + stage * kStageBytesA, &tmap_aux, &full_bar[stage], kb * kBK,
                                    tm * kBM - f.rank * (g.M / f.nranks));
                    } else {
                        tma_load_2d(smem_a + stage * kStageBytesA, &tmap_a, &full_bar[stage], kb * kBK, tm * kBM);
                    }
                    tma_load_2d(smem_b + stage * kStageBytesB, (kMode == Mode::Plain && w.tail) ? &tmap_aux : &tmap_b,
                                &full_bar[stage], kb * kBK, w.col0);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            int stage = 0, acc = 0;
            std::uint32_t phase = 0, acc_phase = 0;
            for (int t = cta; t < total_tiles && *abort_flag == 0; t += num_ctas) {
                const std::uint32_t idesc = make_idesc_bf16(kBM, tile_work<kMode>(t, m_tiles, n_tiles, g, f).bn);
                if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1u)) {
                    gemm_fail(g, kGemmWaitMma, abort_flag);
                    break;
                }
                tcgen05_fence_after_sync();
                const std::uint32_t tmem_d = tmem_base + static_cast<std::uint32_t>(acc * kBN);
                bool failed = false;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase)) {
                        gemm_fail(g, kGemmWaitMma, abort_flag);
                        failed = true;
                        break;
                    }
                    tcgen05_fence_after_sync();
                    const std::uint64_t da = make_smem_desc_sw128(smem_a + stage * kStageBytesA);
                    const std::uint64_t db = make_smem_desc_sw128(smem_b + stage * kStageBytesB);
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k) {
                        umma_bf16(tmem_d, advance_desc_k(da, k), advance_desc_k(db, k), idesc, (kb | k) != 0);
                    }
                    tcgen05_commit(&empty_bar[stage]);  // frees the smem stage when these MMAs finish
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (failed) break;
                tcgen05_commit(&acc_full[acc]);  // accumulator complete
                if (++acc == kAccStages) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
    } else if (warp < kPublisherWarp) {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int quad = warp & 3;                    // TMEM lane quadrant this warp may read
        const int row_in_tile = quad * 32 + lane;
        int acc = 0;
        int epi_slot = 0;
        const bool tracer = threadIdx.x == 64;
        std::uint32_t acc_phase = 0, foreign_tiles = 0;
        if (tracer) trace_stamp(f, 0, &epi_slot, 0);
        for (int t = cta; t < total_tiles; t += num_ctas) {
            const TileWork w = tile_work<kMode>(t, m_tiles, n_tiles, g, f);
            const int tm = w.tm, tn = w.tn, owner = w.owner, bn = w.bn;
            if (*abort_flag != 0) break;
            if (!mbar_wait(&acc_full[acc], acc_phase)) {
                gemm_fail(g, kGemmWaitEpilogue, abort_flag);
                break;
            }
            tcgen05_fence_after_sync();
            if (tracer) trace_stamp(f, 0, &epi_slot, 1);
            const int row = tm * kBM + row_in_tile;
            const int col0 = w.col0;
            bool peer_ok = true;
            __nv_bfloat16* out_row = nullptr;
            int rows_per = 0, tiles_per_owner = 0, tile_in_owner = 0;
            if constexpr (kIsRs<kMode>) {
                rows_per = g.M / f.nranks;
                const int m_per = m_tiles / f.nranks;
                tiles_per_owner = m_per * n_tiles;
                tile_in_owner = (tm - owner * m_per) * n_tiles + tn;
                const int local_row = row - owner * rows_per;
                if (owner != f.rank) {
                    out_row = f.staging[owner] + (static_cast<std::size_t>(f.rank) * rows_per + local_row) * g.N;
                } else {
                    out_row = g.C + static_cast<std::size_t>(local_row) * g.ldc;
                    // all partials of this tile must have landed in my staging
                    if (lane < f.nranks && lane != f.rank) {
                        const std::uint32_t* flag = f.flags[f.rank] + lane * tiles_per_owner + tile_in_owner;
                        const unsigned long long start = dev::global_timer_ns();
                        unsigned spins = 0;
                        while (static_cast<std::int32_t>(dev::ld_acquire_sys(flag) - f.epoch) < 0) {
                            if ((++spins & 63u) == 0u && dev::global_timer_ns() - start > f.timeout_ns) {
                                peer_ok = false;
                                break;
                            }
                        }
                    }
                    peer_ok = __all_sync(0xffffffffu, peer_ok);
                    if (tracer) trace_stamp(f, 0, &epi_slot, 2);
                }
            } else {
                out_row = g.C + static_cast<std::size_t>(row) * g.ldc;
            }
            if (!peer_ok) {
                gemm_fail(g, kGemmWaitPeer, abort_flag);
                break;
            }
            // Pointer to the first of this warp's 32 rows in the destination; rows are g.N apart in
            // every mode (the staging of GemmRs is laid out like the output).
            __nv_bfloat16* warp_out = out_row - static_cast<std::size_t>(lane) * g.N;
            const int warp_row0 = tm * kBM + quad * 32;
            const bool row_ok = row < g.M;
            const bool vec_ok = (g.N % 8) == 0 && (reinterpret_cast<std::uintptr_t>(warp_out) & 15u) == 0;
            unsigned char* stage = smem_epi + (warp - 2) * kEpiWarpBytes;
            const int n_end = col0 + bn < g.N ? col0 + bn : g.N;  // first column that is not this tile's
#pragma unroll 1
            for (int half = 0; half < kBN / kEpiCols; ++half) {
                if (half * kEpiCols >= bn) break;
#pragma unroll 1
                for (int cc = 0; cc < kEpiCols / 32; ++cc) {
                    const int c = half * (kEpiCols / 32) + cc;
                    if (c * 32 >= bn) break;  // a narrower tile has fewer 32-column chunks
                    std::uint32_t r[32];
                    const std::uint32_t taddr = tmem_base + (static_cast<std::uint32_t>(quad * 32) << 16) +
                                                static_cast<std::uint32_t>(acc * kBN + c * 32);
                    tmem_ld_32x32b_x32(taddr, r);
                    tmem_ld_wait();
                    const int col = col0 + c * 32;
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
                    if (g.bias != nullptr && col < g.N) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (col + i < g.N) v[i] += __bfloat162float(g.bias[col + i]);
                        }
                    }
                    if constexpr (kIsRs<kMode>) {
                        if (owner == f.rank && row_ok && col < g.N && col + 32 > g.N) {
                            // ragged right edge: element-wise, only the columns that exist
                            const int local_row = row - owner * rows_per;
                            for (int src = 0; src < f.nranks; ++src) {
                                if (src == f.rank) continue;
                                const __nv_bfloat16* p = f.staging[f.rank] +
                                    (static_cast<std::size_t>(src) * rows_per + local_row) * g.N + col;
#pragma unroll
                                for (int i = 0; i < 32; ++i) {
                                    if (col + i < g.N) {
                                        const unsigned short bits = __ldcg(reinterpret_cast<const unsigned short*>(p) + i);
                                        v[i] += __uint_as_float(static_cast<std::uint32_t>(bits) << 16);
                                    }
                                }
                            }
                        }
                        if (owner == f.rank && row_ok && col + 32 <= g.N) {
                            // add the N-1 staged partials (bf16) of this row segment; all loads of
                            // the chunk are issued before the first add (L2 reads, L1 bypassed: the
                            // data was written by other GPUs during this kernel)
                            const int local_row = row - owner * rows_per;
                            uint4 x[kMaxRanks - 1][4];
#pragma unroll
                            for (int s2 = 0; s2 < kMaxRanks - 1; ++s2) {
                                const int src = s2 < f.rank ? s2 : s2 + 1;   // every rank but mine
                                if (src < f.nranks) {
                                    const uint4* p = reinterpret_cast<const uint4*>(
                                        f.staging[f.rank] + (static_cast<std::size_t>(src) * rows_per + local_row) * g.N + col);
#pragma unroll
                                    for (int q = 0; q < 4; ++q) x[s2][q] = __ldcg(p + q);
                                }
                            }
#pragma unroll
                            for (int s2 = 0; s2 < kMaxRanks - 1; ++s2) {
                                if ((s2 < f.rank ? s2 : s2 + 1) < f.nranks) {
#pragma unroll
                                    for (int q = 0; q < 4; ++q) {
                                        const std::uint32_t w[4] = {x[s2][q].x, x[s2][q].y, x[s2][q].z, x[s2][q].w};
#pragma unroll
                                        for (int i = 0; i < 4; ++i) {
                                            v[q * 8 + 2 * i] += __uint_as_float(w[i] << 16);
                                            v[q * 8 + 2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
                                        }
                                    }
                                }
                            }
                        }
                    }
                    // bf16, into this warp's staging rows; 16-byte chunks are XOR-swizzled by the row
                    // so that neither this write nor the row-wise read-out below conflicts on banks
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint4 o;
                        std::uint32_t* ow = reinterpret_cast<std::uint32_t*>(&o);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const __nv_bfloat162 h = __floats2bfloat162_rn(v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1]);
                            ow[i] = *reinterpret_cast<const std::uint32_t*>(&h);
                        }
                        if (kMode == Mode::GemmRsTma && owner != f.rank) {
                            // layout of two 64-column boxes with the 128-byte swizzle: box, row, chunk ^ (row % 8)
                            const int gch = cc * 4 + q;
                            *reinterpret_cast<uint4*>(stage + (gch >> 3) * kTmaBoxBytes + lane * 128 +
                                                      (((gch & 7) ^ (lane & 7)) << 4)) = o;
                        } else {
                            const int chunk = (cc * 4 + q) ^ (lane & 15);
                            *reinterpret_cast<uint4*>(stage + lane * kEpiRowBytes + chunk * 16) = o;
                        }
                    }
                }
                if (kMode == Mode::GemmRsTma && owner != f.rank) {
                    // every lane makes its shared-memory writes visible to the TMA unit, then one lane sends
                    // the warp's 32 rows x 128 columns as two tensor stores into the owner's staging
                    fence_proxy_async_shared();
                    __syncwarp();
                    if (lane == 0) {
                        const int x = col0 + half * kEpiCols;
                        const int y = f.rank * rows_per + (warp_row0 - owner * rows_per);
                        if (x < n_end) tma_store_2d(&peer_maps.m[owner], stage, x, y);
                        if (x + 64 < n_end) tma_store_2d(&peer_maps.m[owner], stage + kTmaBoxBytes, x + 64, y);
                        bulk_commit_group();
                        bulk_wait_group_read_all();  // the stage is rewritten by the next pass
                    }
                    __syncwarp();
                    continue;
                }
                __syncwarp();
                // read-out: one warp store covers two rows of 256 contiguous bytes each
#pragma unroll 4
                for (int i = 0; i < 16; ++i) {
                    const int rr = 2 * i + (lane >> 4);
                    const int pch = lane & 15;
                    const int lch = pch ^ (rr & 15);
                    const uint4 val = *reinterpret_cast<const uint4*>(stage + rr * kEpiRowBytes + pch * 16);
                    const int gcol = col0 + half * kEpiCols + lch * 8;
                    if (warp_row0 + rr < g.M && gcol < n_end) {
                        __nv_bfloat16* dst = warp_out + static_cast<std::size_t>(rr) * g.N + gcol;
                        if (vec_ok && gcol + 8 <= n_end) {
                            dev::Vec16 o;
                            o.w[0] = val.x; o.w[1] = val.y; o.w[2] = val.z; o.w[3] = val.w;
                            dev::st_vec(dst, o);
                        } else {
                            const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&val);
#pragma unroll
                            for (int k = 0; k < 8; ++k) {
                                if (gcol + k < n_end) dst[k] = e[k];
                            }
                        }
                    }
                }
                __syncwarp();
            }
            // accumulator drained: hand it back to the MMA warp
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc]);
            if (tracer) trace_stamp(f, 0, &epi_slot, 3);
            if constexpr (kIsRs<kMode>) {
                if (owner != f.rank) {
                    // The tile's flag follows the stores of all four epilogue warps: each warp arrives on
                    // epi_bar after its stores and goes on to the next tile; the publisher warp waits for the
                    // four arrivals and publishes the flag with release semantics.  The fence that store
                    // implies waits for every remote store of the tile to be acknowledged (microseconds over
                    // NVLink), which is why no epilogue warp executes it.
                    bool ok = true;
                    if (lane == 0) {
                        if (kMode == Mode::GemmRsTma) {
                            // tensor stores are asynchronous: they must have completed, and be ordered before
                            // ordinary memory operations, before this warp counts as done
                            bulk_wait_group_all();
                            fence_proxy_async_all();
                            __threadfence_system();
                        }
                        const unsigned long long start = dev::global_timer_ns();
                        unsigned spins = 0;
                        while (*epi_seen < foreign_tiles) {
                            if ((++spins & 63u) == 0u &&
                                (*abort_flag != 0 || dev::global_timer_ns() - start > f.timeout_ns)) {
                                ok = false;
                                break;
                            }
                        }
                        if (ok) mbar_arrive(epi_bar);
                    }
                    ++foreign_tiles;
                    if (!__all_sync(0xffffffffu, ok)) {
                        gemm_fail(g, kGemmWaitEpilogue, abort_flag);
                        break;
                    }
                }
            }
            if (++acc == kAccStages) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
    } else if (warp == kPublisherWarp) {
        // ------------------------------------------------------------ GemmRs: tile-flag publisher
        if constexpr (kIsRs<kMode>) {
            if (lane == 0) {
                const int tiles_per_owner = (m_tiles / f.nranks) * n_tiles;
                int pub_slot = 0;
                std::uint32_t phase = 0, seen = 0;
                for (int t = cta; t < total_tiles; t += num_ctas) {
                    int tm, tn, owner;
                    tile_coords<kMode>(t, m_tiles, n_tiles, f, &tm, &tn, &owner);
                    if (owner == f.rank) continue;
                    const unsigned long long start = dev::global_timer_ns();
                    unsigned spins = 0;
                    bool ok = true;
                    while (!mbar_try_wait(epi_bar, phase)) {
                        if ((++spins & 63u) == 0u &&
                            (*abort_flag != 0 || dev::global_timer_ns() - start > f.timeout_ns)) {
                            ok = false;
                            break;
                        }
                    }
                    if (!ok) {
                        if (*abort_flag == 0) gemm_fail(g, kGemmWaitEpilogue, abort_flag);
                        break;
                    }
                    *epi_seen = ++seen;
                    phase ^= 1u;
                    trace_stamp(f, 1, &pub_slot, 7);
                    const int tile_in_owner = (tm - owner * (m_tiles / f.nranks)) * n_tiles + tn;
                    dev::st_release_sys(f.flags[owner] + f.rank * tiles_per_owner + tile_in_owner, f.epoch);
                    trace_stamp(f, 1, &pub_slot, 4);
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after_sync();
        tmem_dealloc<kTmemCols>(tmem_base);
    }
}

}  // namespace nano_nccl::gemm
