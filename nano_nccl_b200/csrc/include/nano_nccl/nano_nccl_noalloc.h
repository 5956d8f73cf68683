/* An AllReduce entry point for callers that must not allocate device memory.
 *
 * This function has no counterpart in the reference library.
 *
 * Who needs it: code that runs where cudaMalloc / cudaFree are off limits or would deadlock —
 * a host callback or a thread that holds a lock the CUDA allocator also takes, a process whose
 * device memory is entirely owned by a caching pool it may not bypass, a component that has been
 * handed a fixed memory budget and audited for "no allocation after start-up", or a region that is
 * being recorded into a CUDA graph elsewhere in the process (cudaMalloc is not legal on a capturing
 * thread).  The regular single-GPU emulation entry point (nano_nccl_emu_create + nano_nccl_emu_
 * all_reduce) allocates its arenas with cudaMalloc; this variant runs the same one-shot AllReduce
 * kernel with all of its scratch memory — staging areas, signal pads, per-block counters, status
 * words — inside one fixed array that is part of the library image.
 *
 * What it does: reduces `nranks` equally sized buffers that live on the current device as if each
 * belonged to one rank of a communicator: dsts[r][i] = op over k of srcs[k][i], for every r.
 * All "ranks" run in one cooperative launch on `stream`; the call returns after enqueueing.
 *
 * Limits (fixed at build time):
 *   - nranks from 1 to NANO_NCCL_NOALLOC_MAX_RANKS (8);
 *   - count from 1 to NANO_NCCL_NOALLOC_MAX_COUNT (4 Mi elements) per buffer;
 *   - the scratch array takes NANO_NCCL_NOALLOC_SCRATCH_BYTES (about 16.6 MiB) of device memory on
 *     every GPU on which this library's device code gets loaded, until the process exits, used or
 *     not.  The CUDA runtime loads device code lazily by default: the array (and the code of each
 *     kernel variant) is then placed on a device by the first call that needs it there, and that
 *     placement is an allocation made by the driver on this library's behalf.
 * Requests beyond the limits are refused with NANO_NCCL_STATUS_INVALID_ARGUMENT and a message in
 * nano_nccl_get_last_error(); nothing is launched.
 *
 * Rules for callers:
 *   - The first call on each device looks up the device address of the scratch array
 *     (cudaGetSymbolAddress, with that device current), and the first call of each (dtype,
 *     operator) pair makes the driver load that kernel.  Make those first calls at start-up, once
 *     per device and per variant you will use, before the no-allocation regime begins and before
 *     any stream capture begins on the calling thread; later calls allocate nothing anywhere.
 *   - Every call uses the same scratch array, and the array keeps whatever the previous call left
 *     in it; the control part (signal pads, counters, status) is cleared on `stream` at the start
 *     of every call.  Two calls whose kernels may overlap on the GPU (different streams, or the
 *     same buffers used from two threads) race on the scratch and give wrong results: order them.
 *   - Buffers must not overlap each other; srcs[r] == dsts[r] is not allowed.
 *   - A wait that runs out inside the kernel (it cannot happen unless the launch was starved of
 *     SMs for seconds) ends the kernel early and leaves the outputs incomplete.  The kernel notes
 *     that in status words inside the scratch array; nano_nccl_all_reduce_local_noalloc_status()
 *     waits for `stream` and reads them back (into caller memory, without allocating).  Call it
 *     before the next AllReduce on the device, which clears the words.
 * It calls no cudaMalloc, cudaFree, cudaHostAlloc or any allocating routine of another library. */
#ifndef NANO_NCCL_NANO_NCCL_NOALLOC_H_
#define NANO_NCCL_NANO_NCCL_NOALLOC_H_

#include "nano_nccl/nano_nccl.h"

#ifdef __cplusplus
extern "C" {
#endif

#define NANO_NCCL_NOALLOC_MAX_RANKS 8
#define NANO_NCCL_NOALLOC_MAX_COUNT (4u * 1024u * 1024u)
/* 8 ranks x (64 KiB signal pads + 2 MiB staging) + counters and status words */
#define NANO_NCCL_NOALLOC_SCRATCH_BYTES (8u * (64u * 1024u + 2u * 1024u * 1024u) + 64u * 1024u)

nano_nccl_status_t nano_nccl_all_reduce_local_noalloc(const void* const* srcs, void* const* dsts,
                                                      int nranks, size_t count,
                                                      nano_nccl_dtype_t dtype,
                                                      nano_nccl_redop_t redop, cudaStream_t stream);

/* Synchronous: waits for `stream`, then copies the status words of the last call on the current device into
 * words[0..3] = {code, peer rank, phase, block}; all zero and NANO_NCCL_STATUS_SUCCESS when every wait of that
 * call was satisfied, the first failing rank's words and NANO_NCCL_STATUS_ERROR otherwise.  Allocates nothing.
 * No counterpart in the reference. */
nano_nccl_status_t nano_nccl_all_reduce_local_noalloc_status(cudaStream_t stream, uint32_t words[4]);

#ifdef __cplusplus
}
#endif

#endif /* NANO_NCCL_NANO_NCCL_NOALLOC_H_ */
