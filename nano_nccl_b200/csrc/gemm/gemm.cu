#include "gemm/gemm.h"

#include "core/buffer.h"
#include "core/driver.h"
#include "core/env.h"
#include "core/error.h"
#include "gemm/gemm_kernel.cuh"

#include <cstdlib>
#include <map>
#include <mutex>

namespace nano_nccl {

using namespace gemm;

namespace {

// bf16 row-major [rows][cols] -> 2-D tensor map with a (64 x box_rows) box and 128-byte swizzle.
CUtensorMap make_tmap(const void* base, int rows, int cols, int box_rows) {
    NANO_REQUIRE_ARG((reinterpret_cast<std::uintptr_t>(base) & 15u) == 0, "GEMM operand must be 16-byte aligned");
    NANO_REQUIRE_ARG(cols % 8 == 0, "GEMM inner dimension %d must be a multiple of 8", cols);
    CUtensorMap map;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem_strides[2] = {1, 1};
    CU_CHECK_THROW(driver::api().TensorMapEncodeTiled(
        &map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    return map;
}

// bf16 row-major [rows][cols] in this GPU's or a peer's memory, as the target of 64 x 32 tile stores
// whose shared-memory source uses the 128-byte swizzle.
CUtensorMap make_store_tmap(const void* base, int rows, int cols) {
    NANO_REQUIRE_ARG((reinterpret_cast<std::uintptr_t>(base) & 15u) == 0 && cols % 8 == 0,
                     "tile-store target must be 16-byte aligned with a row length that is a multiple of 8");
    CUtensorMap map;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
    const cuuint32_t box[2] = {64, 32};
    const cuuint32_t elem_strides[2] = {1, 1};
    CU_CHECK_THROW(driver::api().TensorMapEncodeTiled(
        &map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    return map;
}

struct DeviceState {
    MappedBuffer<int> error;
    int sms = 0;
    bool attrs_set = false;
};

DeviceState& device_state(int device) {
    static std::mutex mutex;
    static std::map<int, DeviceState> states;
    std::lock_guard<std::mutex> lock(mutex);
    auto it = states.find(device);
    if (it == states.end()) {
        DeviceState st;
        st.error = MappedBuffer<int>(4);
        CUDA_CHECK_THROW(cudaDeviceGetAttribute(&st.sms, cudaDevAttrMultiProcessorCount, device));
        it = states.emplace(device, std::move(st)).first;
    }
    DeviceState& st = it->second;
    if (!st.attrs_set) {
        CUDA_CHECK_THROW(cudaFuncSetAttribute(gemm_bf16_kernel<Mode::Plain>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes)));
        CUDA_CHECK_THROW(cudaFuncSetAttribute(gemm_bf16_kernel<Mode::GemmRs>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes)));
        CUDA_CHECK_THROW(cudaFuncSetAttribute(gemm_bf16_kernel<Mode::AgGemm>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes)));
        CUDA_CHECK_THROW(cudaFuncSetAttribute(gemm_bf16_kernel<Mode::GemmRsTma>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes)));
        st.attrs_set = true;
    }
    return st;
}

int current_device() {
    int d = 0;
    CUDA_CHECK_THROW(cudaGetDevice(&d));
    return d;
}

}  // namespace

int gemm_pick_tile_width(int m_tiles, int N, int ctas, int granule) {
    const auto setting = env::get("NANO_NCCL_GEMM_BN");
    if (!setting || setting->empty()) return kBN;
    if (*setting != "auto") {
        const long v = std::strtol(setting->c_str(), nullptr, 10);
        NANO_REQUIRE_ARG(v >= 32 && v <= kBN && v % granule == 0,
                         "NANO_NCCL_GEMM_BN must be 'auto' or a multiple of %d in [32, %d]", granule, kBN);
        return static_cast<int>(v);
    }
    int best = kBN;
    long best_cost = -1;
    for (int bn = kBN; bn >= 192; bn -= 32) {  // narrower tiles lose too much operand reuse to be picked blindly
        if (bn % granule != 0) continue;
        const long tiles = static_cast<long>(m_tiles) * ((N + bn - 1) / bn);
        const long waves = (tiles + ctas - 1) / ctas;
        const long cost = waves * bn;
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

GemmTailSplit gemm_pick_tail_split(int tiles, int ctas, int bn) {
    GemmTailSplit none;
    none.first_tile = tiles;
    if (!env::flag("NANO_NCCL_GEMM_TAIL", true) || ctas <= 0 || tiles <= ctas) return none;
    const int rest = tiles % ctas;
    if (rest == 0 || rest * 2 > ctas) return none;
    for (int piece = 32; piece <= 128; piece *= 2) {
        if (bn % piece != 0 || piece >= bn) continue;
        if (static_cast<long>(rest) * (bn / piece) <= ctas) {
            GemmTailSplit split;
            split.first_tile = tiles - rest;
            split.piece_bn = piece;
            return split;
        }
    }
    return none;
}

void gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, cudaStream_t stream,
               int max_ctas) {
    NANO_REQUIRE_ARG(A != nullptr && B != nullptr && C != nullptr, "GEMM operands must be non-null");
    NANO_REQUIRE_ARG(M > 0 && N > 0 && K > 0, "GEMM sizes must be positive");
    DeviceState& st = device_state(current_device());
    const int sms_avail = max_ctas > 0 ? std::min(max_ctas, st.sms) : st.sms;
    const int bn = gemm_pick_tile_width((M + kBM - 1) / kBM, N, sms_avail, 32);
    const CUtensorMap ta = make_tmap(A, M, K, kBM);
    const CUtensorMap tb = make_tmap(B, N, K, bn);
    GemmArgs g;
    g.bn = bn;
    g.M = M; g.N = N; g.K = K;
    g.C = static_cast<__nv_bfloat16*>(C);
    g.ldc = N;
    g.bias = static_cast<const __nv_bfloat16*>(bias);
    g.error = st.error.device();
    FusedArgs f;
    const int tiles = ((M + kBM - 1) / kBM) * ((N + bn - 1) / bn);
    int grid = max_ctas > 0 ? std::min(max_ctas, st.sms) : st.sms;
    grid = std::max(1, std::min(grid, tiles));
    // the last, partly filled round of tiles is cut into narrow column pieces (their own tensor map of B)
    const GemmTailSplit tail = gemm_pick_tail_split(tiles, grid, bn);
    g.tail_first = tail.first_tile;
    g.tail_bn = tail.piece_bn;
    const CUtensorMap tb_tail = tail.piece_bn > 0 ? make_tmap(B, N, K, tail.piece_bn) : tb;
    gemm_bf16_kernel<Mode::Plain><<<grid, kGemmThreads, kSmemBytes, stream>>>(ta, tb, tb_tail, g, f, PeerMaps{});
    CUDA_CHECK_THROW(cudaGetLastError());
}

int gemm_last_error(int device) { return *static_cast<volatile int*>(device_state(device).error.host()); }
void gemm_clear_error(int device) { device_state(device).error.host()[0] = 0; }

// ------------------------------------------------------------------------------------------------
struct FusedGemmContext::State {
    int rank = 0, nranks = 1, device = 0;
    std::size_t rs_bytes = 0, ag_bytes = 0;
    // two parities of everything: a peer may be one call ahead
    void* rs_staging[2] = {nullptr, nullptr};
    void* ag_gathered[2] = {nullptr, nullptr};
    void* flags = nullptr;  // u32: [parity-independent] rs flags then ag flags
    std::size_t rs_flag_words = 0, ag_flag_words = 0;
    std::uint32_t epoch = 0;
    unsigned long long timeout_ns = 20'000'000'000ull;
    RawDeviceBuffer trace;       // NANO_NCCL_GEMM_TRACE=1: per-CTA time line of the last fused call
    std::size_t trace_words = 0;
    int ag_push_parts = 0;       // NANO_NCCL_AG_PUSH_PARTS: units per 128-row block (power of two, 1..32); 0 = default
    int ag_push_ctas = 0;        // NANO_NCCL_AG_PUSH_CTAS: CTAs that only move data in AllGather->GEMM; 0 = default
    bool ag_tma_push = false;    // NANO_NCCL_AG_GEMM_TMA=1: AllGather->GEMM pushers use TMA bulk copies
    bool rs_tma_stores = false;  // NANO_NCCL_GEMM_RS_TMA=1: remote epilogue through TMA tensor stores
};

namespace {
constexpr std::size_t kMaxFlagWords = 64 * 1024;  // per kind
}

FusedGemmContext::FusedGemmContext(Communicator& comm, std::size_t max_rs_bytes, std::size_t max_ag_bytes)
    : s_(new State()), comm_(comm) {
    s_->rank = comm.rank();
    s_->nranks = comm.global_rank_count();
    s_->device = comm.device();
    s_->rs_bytes = max_rs_bytes;
    s_->ag_bytes = max_ag_bytes;
    s_->rs_flag_words = kMaxFlagWords;
    s_->ag_flag_words = kMaxFlagWords;
    s_->timeout_ns = static_cast<unsigned long long>(
                         env::integer("NANO_NCCL_WAIT_TIMEOUT_US", 20'000'000, 1000, 3'600'000'000ll)) * 1000ull;
    s_->rs_tma_stores = env::flag("NANO_NCCL_GEMM_RS_TMA", false);
    s_->ag_tma_push = env::flag("NANO_NCCL_AG_GEMM_TMA", false);
    s_->ag_push_parts = static_cast<int>(env::integer("NANO_NCCL_AG_PUSH_PARTS", 0, 0, kMaxPushParts));
    s_->ag_push_ctas = static_cast<int>(env::integer("NANO_NCCL_AG_PUSH_CTAS", 0, 0, 64));
    NANO_REQUIRE_ARG((s_->ag_push_parts & (s_->ag_push_parts - 1)) == 0, "NANO_NCCL_AG_PUSH_PARTS must be a power of two");
    if (env::flag("NANO_NCCL_GEMM_TRACE", false)) {
        int sms = 0;
        CUDA_CHECK_THROW(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, s_->device));
        s_->trace_words = static_cast<std::size_t>(sms + 64) * 2 * kTraceSlots;
        s_->trace = RawDeviceBuffer(s_->device, s_->trace_words * sizeof(unsigned long long), true);
    }
    for (int p = 0; p < 2; ++p) {
        if (max_rs_bytes != 0) s_->rs_staging[p] = comm.symmetric_alloc(max_rs_bytes);
        if (max_ag_bytes != 0) s_->ag_gathered[p] = comm.symmetric_alloc(max_ag_bytes);
    }
    s_->flags = comm.symmetric_alloc((s_->rs_flag_words + s_->ag_flag_words) * sizeof(std::uint32_t));
}

FusedGemmContext::~FusedGemmContext() {
    // Symmetric segments are released with the communicator; freeing here would need a collective.
}

void FusedGemmContext::gemm_rs(const void* A, const void* W, void* out, int M, int N, int Kp, cudaStream_t stream) {
    State& s = *s_;
    const int R = s.nranks;
    NANO_REQUIRE_ARG(M > 0 && N > 0 && Kp > 0 && M % (R * kBM) == 0, "gemm_rs: M=%d must be a multiple of ranks*128", M);
    NANO_REQUIRE_ARG(N % 8 == 0 && Kp % 8 == 0, "gemm_rs: N and K must be multiples of 8");
    NANO_REQUIRE_ARG(static_cast<std::size_t>(M) * N * 2 <= s.rs_bytes, "gemm_rs: workspace too small");
    const int bn = gemm_pick_tile_width(M / kBM, N, device_state(s.device).sms, s.rs_tma_stores ? 64 : 32);
    const int m_per = M / R / kBM, n_tiles = (N + bn - 1) / bn;
    NANO_REQUIRE_ARG(static_cast<std::size_t>(R) * m_per * n_tiles <= s.rs_flag_words, "gemm_rs: too many tiles for the flag area");
    CUDA_CHECK_THROW(cudaSetDevice(s.device));
    DeviceState& st = device_state(s.device);
    const CUtensorMap ta = make_tmap(A, M, Kp, kBM);
    const CUtensorMap tb = make_tmap(W, N, Kp, bn);
    GemmArgs g;
    g.bn = bn;
    g.M = M; g.N = N; g.K = Kp;
    g.C = static_cast<__nv_bfloat16*>(out);
    g.ldc = N;
    g.error = st.error.device();
    FusedArgs f;
    f.rank = s.rank;
    f.nranks = R;
    f.epoch = ++s.epoch;
    f.timeout_ns = s.timeout_ns;
    if (s.trace_words != 0) {
        CUDA_CHECK_THROW(cudaMemsetAsync(s.trace.data(), 0, s.trace_words * sizeof(unsigned long long), stream));
        f.trace = static_cast<unsigned long long*>(s.trace.data());
    }
    const int parity = static_cast<int>(f.epoch & 1u);
    for (int r = 0; r < R; ++r) {
        f.staging[r] = static_cast<__nv_bfloat16*>(comm_.peer_pointer(s.rs_staging[parity], r));
        f.flags[r] = static_cast<std::uint32_t*>(comm_.peer_pointer(s.flags, r));
    }
    const int tiles = (M / kBM) * n_tiles;
    const int grid = std::max(1, std::min(st.sms, tiles));
    if (s.rs_tma_stores) {
        // one tensor map per rank over its staging [M][N] (rank-major blocks of rows), boxes of 64 x 32
        PeerMaps maps{};
        for (int r = 0; r < R; ++r) maps.m[r] = make_store_tmap(f.staging[r], M, N);
        gemm_bf16_kernel<Mode::GemmRsTma><<<grid, kGemmThreads, kSmemBytes, stream>>>(ta, tb, ta, g, f, maps);
    } else {
        gemm_bf16_kernel<Mode::GemmRs><<<grid, kGemmThreads, kSmemBytes, stream>>>(ta, tb, ta, g, f, PeerMaps{});
    }
    CUDA_CHECK_THROW(cudaGetLastError());
}

void FusedGemmContext::ag_gemm(const void* x_shard, const void* W, void* out, int M, int Np, int K,
                               cudaStream_t stream, int push_ctas) {
    State& s = *s_;
    const int R = s.nranks;
    NANO_REQUIRE_ARG(M > 0 && Np > 0 && K > 0 && M % (R * kBM) == 0, "ag_gemm: M=%d must be a multiple of ranks*128", M);
    NANO_REQUIRE_ARG(K % 8 == 0, "ag_gemm: K must be a multiple of 8");
    NANO_REQUIRE_ARG(static_cast<std::size_t>(M) * K * 2 <= s.ag_bytes, "ag_gemm: workspace too small");
    const int blocks = M / R / kBM;
    NANO_REQUIRE_ARG(static_cast<std::size_t>(R) * blocks * kMaxPushParts <= s.ag_flag_words,
                     "ag_gemm: too many row blocks for the flag area");
    CUDA_CHECK_THROW(cudaSetDevice(s.device));
    DeviceState& st = device_state(s.device);
    FusedArgs f;
    f.rank = s.rank;
    f.nranks = R;
    f.epoch = ++s.epoch;
    f.timeout_ns = s.timeout_ns;
    if (s.trace_words != 0) {
        CUDA_CHECK_THROW(cudaMemsetAsync(s.trace.data(), 0, s.trace_words * sizeof(unsigned long long), stream));
        f.trace = static_cast<unsigned long long*>(s.trace.data());
    }
    const int parity = static_cast<int>(f.epoch & 1u);
    for (int r = 0; r < R; ++r) {
        f.gathered[r] = static_cast<__nv_bfloat16*>(comm_.peer_pointer(s.ag_gathered[parity], r));
        f.flags[r] = static_cast<std::uint32_t*>(comm_.peer_pointer(s.flags, r)) + s.rs_flag_words;
    }
    f.gathered_mc = static_cast<__nv_bfloat16*>(comm_.multicast_pointer(s.ag_gathered[parity]));
    f.shard = static_cast<const __nv_bfloat16*>(x_shard);
    // Pushers take SMs from the GEMM for the whole kernel, so as few as keep the transfer ahead of the MMAs: with 2
    // ranks the own half of the rows (half of the GEMM) is computed before the first remote block is needed and only
    // one peer is written, so 8 are enough; from 4 ranks on 16.  NANO_NCCL_AG_PUSH_CTAS overrides.
    if (push_ctas <= 0) push_ctas = s.ag_push_ctas > 0 ? s.ag_push_ctas : (R == 2 ? 8 : 16);
    push_ctas = std::min(push_ctas, std::max(1, st.sms / 2));
    if (R == 1) push_ctas = 0;
    f.push_ctas = push_ctas;
    // Units per 128-row block.  With 2, 16 pushers work on 8 blocks at once, so at 8 GPUs the whole shard arrives
    // together and the GEMM of the remote rows waits for all of it; with 8 (the default) they work through the blocks
    // in order (two blocks in flight) and the GEMM follows the transfer.  Measured on 8 B200, 8192 x 1792 x 4096:
    // 164 us against 182 us (2 GPUs: 395 against 389 us); more units cost a flag round trip each.
    // NANO_NCCL_AG_PUSH_PARTS selects.
    int parts = s.ag_push_parts > 0 ? s.ag_push_parts : 8;
    while (parts > 1 && parts > push_ctas) parts /= 2;
    f.push_parts = std::max(1, parts);
    f.push_tma = s.ag_tma_push && (static_cast<std::size_t>(K) * 2) % 16 == 0 ? 1 : 0;
    const CUtensorMap ta = make_tmap(s.ag_gathered[parity], M, K, kBM);
    const CUtensorMap tshard = make_tmap(x_shard, M / R, K, kBM);
    const int bn = gemm_pick_tile_width(M / kBM, Np, std::max(1, st.sms - push_ctas), 32);
    const CUtensorMap tb = make_tmap(W, Np, K, bn);
    GemmArgs g;
    g.bn = bn;
    g.M = M; g.N = Np; g.K = K;
    g.C = static_cast<__nv_bfloat16*>(out);
    g.ldc = Np;
    g.error = st.error.device();
    const int tiles = (M / kBM) * ((Np + bn - 1) / bn);
    const int grid = push_ctas + std::max(1, std::min(st.sms - push_ctas, tiles));
    gemm_bf16_kernel<Mode::AgGemm><<<grid, kGemmThreads, kSmemBytes, stream>>>(ta, tb, tshard, g, f, PeerMaps{});
    CUDA_CHECK_THROW(cudaGetLastError());
}

std::size_t FusedGemmContext::read_trace(unsigned long long* out, std::size_t max_words) {
    State& s = *s_;
    if (s.trace_words == 0) return 0;
    const std::size_t n = std::min(max_words, s.trace_words);
    CUDA_CHECK_THROW(cudaSetDevice(s.device));
    CUDA_CHECK_THROW(cudaDeviceSynchronize());
    CUDA_CHECK_THROW(cudaMemcpy(out, s.trace.data(), n * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    return n;
}

}  // namespace nano_nccl
