/* C ABI extensions that have no counterpart in the reference: creating a communicator from a TCP
 * rendezvous or from caller-supplied control callbacks, symmetric memory, algorithm selection,
 * the fused tensor-parallel GEMMs, and observability counters. */
#ifndef NANO_NCCL_NANO_NCCL_EXT_H_
#define NANO_NCCL_NANO_NCCL_EXT_H_

#include "nano_nccl/nano_nccl.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t nano_nccl_algo_t;
enum {
    NANO_NCCL_ALGO_AUTO = 0,
    NANO_NCCL_ALGO_ONESHOT = 1,
    NANO_NCCL_ALGO_TWOSHOT = 2,
    NANO_NCCL_ALGO_NVLS = 3,
    NANO_NCCL_ALGO_RING = 4,
};

typedef struct NanoNcclExtConfig {
    int device;
    nano_nccl_transport_t transport;
    nano_nccl_algo_t algo;
    int enable_multicast;      /* -1 default, 0 off, 1 on */
    int64_t wait_timeout_us;   /* 0 = default */
    int relaxed_validation;    /* 1: accept the default stream and exact in-place all_reduce */
} nano_nccl_ext_config_t;

/* Rendezvous over TCP: rank 0 listens on addr:port. */
nano_nccl_status_t nano_nccl_create_tcp_communicator(const char* addr, int port, int rank,
                                                     int size, const nano_nccl_ext_config_t* config,
                                                     nano_nccl_communicator_t** communicator);

/* Rendezvous over a caller-provided all-gather of `bytes` per rank (blocking, same order on all
 * ranks).  `user` is passed back unchanged.  The callback must stay valid until destroy. */
typedef void (*nano_nccl_allgather_fn)(void* user, const void* in, void* out, size_t bytes);
nano_nccl_status_t nano_nccl_create_callback_communicator(nano_nccl_allgather_fn allgather,
                                                          void* user, int rank, int size,
                                                          const nano_nccl_ext_config_t* config,
                                                          nano_nccl_communicator_t** communicator);

/* Exercises a caller-provided all-gather without touching a GPU: returns 0 when three rounds of
 * different sizes come back rank-major and intact, a positive code otherwise. */
int nano_nccl_bootstrap_selftest(nano_nccl_allgather_fn allgather, void* user, int rank, int size);

nano_nccl_status_t nano_nccl_rank(const nano_nccl_communicator_t* communicator, int* rank);
nano_nccl_status_t nano_nccl_multicast_available(const nano_nccl_communicator_t* communicator,
                                                 int* available);
nano_nccl_status_t nano_nccl_set_algo(nano_nccl_communicator_t* communicator,
                                      nano_nccl_algo_t algo);
/* ctas > 0: every collective uses exactly that many CTAs (tuning sweeps); 0: tuner table. */
nano_nccl_status_t nano_nccl_set_grid_override(nano_nccl_communicator_t* communicator, int ctas);
nano_nccl_status_t nano_nccl_last_algo(const nano_nccl_communicator_t* communicator,
                                       nano_nccl_algo_t* algo);

/* Collective: all ranks call with the same size, in the same order. */
nano_nccl_status_t nano_nccl_symmetric_alloc(nano_nccl_communicator_t* communicator, size_t bytes,
                                             void** ptr);
nano_nccl_status_t nano_nccl_symmetric_free(nano_nccl_communicator_t* communicator, void* ptr);
/* Collective: registers a caller-owned device buffer (same size on every rank, 16-byte aligned) so that the
 * zero-copy kernels apply to it; memory from the virtual-memory API or stream-ordered pools is refused. */
nano_nccl_status_t nano_nccl_register_buffer(nano_nccl_communicator_t* communicator, void* ptr, size_t bytes);
nano_nccl_status_t nano_nccl_deregister_buffer(nano_nccl_communicator_t* communicator, void* ptr);
nano_nccl_status_t nano_nccl_peer_pointer(const nano_nccl_communicator_t* communicator,
                                          const void* ptr, int peer_rank, void** peer_ptr);
nano_nccl_status_t nano_nccl_multicast_pointer(const nano_nccl_communicator_t* communicator,
                                               const void* ptr, void** mc_ptr);
nano_nccl_status_t nano_nccl_barrier(nano_nccl_communicator_t* communicator, cudaStream_t stream);

typedef struct NanoNcclStats {
    uint64_t launches, oneshot, twoshot, nvls, ring, zero_copy, local_only, pipelined;
} nano_nccl_stats_t;
nano_nccl_status_t nano_nccl_get_stats(const nano_nccl_communicator_t* communicator,
                                       nano_nccl_stats_t* stats);

/* ---- single-GPU emulation of an N-rank communicator (testing aid) ----
 * All ranks' arenas live on one GPU and one cooperative launch runs every rank's blocks, so the
 * peer-to-peer kernels can be exercised, and the bounded device wait observed, on one GPU. */
typedef struct NanoNcclEmulatedCluster nano_nccl_emulated_cluster_t;
nano_nccl_status_t nano_nccl_emu_create(int device, int nranks, int64_t wait_timeout_us,
                                        nano_nccl_emulated_cluster_t** cluster);
nano_nccl_status_t nano_nccl_emu_destroy(nano_nccl_emulated_cluster_t* cluster);
/* srcs / dsts: arrays of nranks device pointers. algo: ONESHOT or TWOSHOT. */
nano_nccl_status_t nano_nccl_emu_all_reduce(nano_nccl_emulated_cluster_t* cluster,
                                            const void* const* srcs, void* const* dsts, size_t count,
                                            nano_nccl_dtype_t dtype, nano_nccl_redop_t redop,
                                            nano_nccl_algo_t algo, int max_grid, cudaStream_t stream);
nano_nccl_status_t nano_nccl_emu_reduce_scatter(nano_nccl_emulated_cluster_t* cluster,
                                                const void* const* srcs, void* const* dsts,
                                                size_t recv_count, nano_nccl_dtype_t dtype,
                                                nano_nccl_redop_t redop, int max_grid,
                                                cudaStream_t stream);
nano_nccl_status_t nano_nccl_emu_all_gather(nano_nccl_emulated_cluster_t* cluster,
                                            const void* const* srcs, void* const* dsts,
                                            size_t send_count, nano_nccl_dtype_t dtype, int max_grid,
                                            cudaStream_t stream);
/* One rank waits alone for peers that never arrive; returns after launch. */
nano_nccl_status_t nano_nccl_emu_lonely_barrier(nano_nccl_emulated_cluster_t* cluster, int rank,
                                                cudaStream_t stream);
/* words: code, peer, phase, block */
nano_nccl_status_t nano_nccl_emu_status(const nano_nccl_emulated_cluster_t* cluster, int rank,
                                        uint32_t words[4]);
nano_nccl_status_t nano_nccl_emu_clear_status(nano_nccl_emulated_cluster_t* cluster);
nano_nccl_status_t nano_nccl_emu_set_abort(nano_nccl_emulated_cluster_t* cluster, int on);

/* ---- tcgen05 GEMM and fused tensor-parallel GEMM+collective kernels (bf16) ---- */
/* C[M,N] = A[M,K] * B[N,K]^T (+ bias[N]); row-major bf16, fp32 accumulation; K % 8 == 0. */
nano_nccl_status_t nano_nccl_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M,
                                       int N, int K, cudaStream_t stream, int max_ctas);
/* First error recorded by a GEMM kernel on the device (0 none; see gemm_kernel.cuh GemmError). */
int nano_nccl_gemm_last_error(int device);
void nano_nccl_gemm_clear_error(int device);

typedef struct NanoNcclFusedGemm nano_nccl_fused_gemm_t;
/* Collective. max_rs_bytes = M*N*2 of the largest GEMM->ReduceScatter; max_ag_bytes = M*K*2 of the
 * largest AllGather->GEMM input. */
nano_nccl_status_t nano_nccl_fused_gemm_create(nano_nccl_communicator_t* communicator,
                                               size_t max_rs_bytes, size_t max_ag_bytes,
                                               nano_nccl_fused_gemm_t** fused);
nano_nccl_status_t nano_nccl_fused_gemm_destroy(nano_nccl_fused_gemm_t* fused);
/* out[M/R, N] = this rank's rows of sum_r A_r[M,Kp] * W_r[N,Kp]^T */
nano_nccl_status_t nano_nccl_gemm_rs(nano_nccl_fused_gemm_t* fused, const void* A, const void* W,
                                     void* out, int M, int N, int Kp, cudaStream_t stream);
/* out[M, Np] = AllGather(x_shard[M/R, K]) * W[Np, K]^T */
nano_nccl_status_t nano_nccl_ag_gemm(nano_nccl_fused_gemm_t* fused, const void* x_shard, const void* W,
                                     void* out, int M, int Np, int K, cudaStream_t stream,
                                     int push_ctas);

/* Diagnostic time line of the last fused call; only with NANO_NCCL_GEMM_TRACE=1 at nano_nccl_fused_gemm_create.
 * Layout: [cta][role 0 = epilogue, 1 = TMA producer][128] words of (tag << 60) | global-timer nanoseconds. */
nano_nccl_status_t nano_nccl_fused_gemm_read_trace(nano_nccl_fused_gemm_t* fused, unsigned long long* out,
                                                   size_t max_words, size_t* words);

/* ---- tensors in symmetric memory for a framework's caching allocator ----
 * nano_nccl_torch_alloc / nano_nccl_torch_free have the signature torch.cuda.memory.CUDAPluggableAllocator expects.
 * Allocation is a collective of the bound communicator (every rank allocates in the same order); a freed segment is
 * parked and released with the communicator.  Bind NULL to unbind. */
nano_nccl_status_t nano_nccl_allocator_bind(nano_nccl_communicator_t* communicator);
void* nano_nccl_torch_alloc(size_t size, int device, cudaStream_t stream);
void nano_nccl_torch_free(void* ptr, size_t size, int device, cudaStream_t stream);
nano_nccl_status_t nano_nccl_allocator_stats(size_t* live_bytes, size_t* parked_bytes);

/* ---- data movement building blocks (measured by nano_nccl_b200.bench.p2p_bandwidth) ---- */
/* Copies `bytes` (multiple of 16) from src to each of ndst (1..8) destinations, this GPU's or peers' memory,
 * all 16-byte aligned.  engine 0: TMA bulk copies driven by one thread per CTA through `stages` (3..16)
 * shared-memory stages of chunk_bytes; engine 1: vector loads / stores from ctas x 288 threads (chunk_bytes
 * and stages ignored); engine 2: the copy engine, one cudaMemcpyAsync per destination.
 * device_error: a zeroed int in device memory, set to 1 if a bounded wait ran out. */
nano_nccl_status_t nano_nccl_push_copy(int engine, const void* src, void* const* dsts, int ndst, size_t bytes,
                                       int ctas, int chunk_bytes, int stages, int* device_error,
                                       cudaStream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* NANO_NCCL_NANO_NCCL_EXT_H_ */
