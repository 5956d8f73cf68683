// Host API of the tcgen05 GEMM and of the fused tensor-parallel GEMM+collective kernels.
#pragma once

#include "nano_nccl/communicator.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <memory>

namespace nano_nccl {

// C[M,N] = A[M,K] * B[N,K]^T (+ bias[N]); all bf16, row-major, fp32 accumulation.
// K must be a multiple of 8 (16-byte row pitch for TMA); A, B 16-byte aligned.
// max_ctas <= 0: one CTA per SM.
void gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
               cudaStream_t stream, int max_ctas = 0);
// First error code recorded by a GEMM kernel on `device` (0: none).  Read from mapped host memory,
// meaningful after the stream has been synchronised.
int gemm_last_error(int device);
void gemm_clear_error(int device);

// Columns per output tile for a problem of `m_tiles` row tiles and N columns on `ctas` CTAs.  Follows
// NANO_NCCL_GEMM_BN: unset -> 256; a number -> that width; "auto" -> the multiple of `granule` (32, or 64
// when the epilogue writes 64-column boxes) in [192, 256] that needs the least tensor-core time, i.e.
// whole waves of CTAs times the width, ties to the wider tile.  Throws std::invalid_argument on a bad setting.
int gemm_pick_tile_width(int m_tiles, int N, int ctas, int granule = 32);

// Split of the last, partly filled wave of a persistent GEMM.  `tiles` output tiles of `bn` columns walked by
// `ctas` CTAs leave tiles % ctas tiles for a last round in which most CTAs idle; when that remainder is at most
// half the CTAs, its tiles are cut into column pieces of `piece_bn` (128, 64 or 32: the narrowest width whose
// pieces still fit one round) so that the round costs a fraction of a full tile instead of a whole one.
// Returns {first linear tile index of the split part, piece_bn}; piece_bn == 0: no split.
// NANO_NCCL_GEMM_TAIL=0 switches the split off.
struct GemmTailSplit {
    int first_tile = 0;
    int piece_bn = 0;
};
GemmTailSplit gemm_pick_tail_split(int tiles, int ctas, int bn);

// Workspace and flags of the fused kernels for one (M, N, K) problem family on one communicator.
// Collective to construct (symmetric allocations).
class FusedGemmContext {
public:
    // max_rs_bytes: M * N * 2 of the largest GEMM->RS output before scattering;
    // max_ag_bytes: M * K * 2 of the largest gathered activation.
    FusedGemmContext(Communicator& comm, std::size_t max_rs_bytes, std::size_t max_ag_bytes);
    ~FusedGemmContext();

    // Row-parallel: partial[M,N] = A[M,Kp] * W[N,Kp]^T on every rank; out[M/R, N] = rows of
    // sum over ranks owned by this rank.  M % (R * 128) == 0, N % 8 == 0, Kp % 8 == 0.
    void gemm_rs(const void* A, const void* W, void* out, int M, int N, int Kp, cudaStream_t stream);
    // Column-parallel: out[M, Np] = AllGather(x_shard[M/R, K])[M, K] * W[Np, K]^T.
    // M % (R * 128) == 0, K % 8 == 0.
    void ag_gemm(const void* x_shard, const void* W, void* out, int M, int Np, int K, cudaStream_t stream,
                 int push_ctas = 0);

    // Diagnostic time line of the last fused call (NANO_NCCL_GEMM_TRACE=1 when the context is created):
    // for every CTA two rows of 128 words, the epilogue's and the TMA producer's; a word is
    // (tag << 60) | nanoseconds of the GPU's global timer, tags as in gemm_kernel.cuh (FusedArgs::trace).
    // Synchronises the device.  Returns the number of words copied (0 when tracing is off).
    std::size_t read_trace(unsigned long long* out, std::size_t max_words);

private:
    struct State;
    std::unique_ptr<State> s_;
    Communicator& comm_;
};

}  // namespace nano_nccl
