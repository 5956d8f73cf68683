// Plain-data view of a communicator that kernels receive by value, and the layout constants of
// the symmetric arena they index.
//
// Arena layout (identical on every rank, so one offset addresses the same slot everywhere):
//   [ signal pads : kMaxBlocks x kMaxRanks u32 ]  peers store here, the owner polls here
//   [ per-block staging : kMaxBlocks x 2 halves x kHalfBytes ]
// Each CTA index owns its pad row and its staging region on all ranks; a CTA only ever talks to
// the CTA with the same index on the other GPUs.  The two staging halves alternate per launch
// (per-block sequence number), which is what makes back-to-back collectives safe without a
// trailing barrier: a peer can be at most one launch behind when it is written to.
//
// Parity: replaces the reference's per-edge FIFO region and step counters
// (src/transport/simple/connection.h:11-42, protocol.h:16-71).
#pragma once

#include "nano_nccl/types.h"

#include <cstddef>
#include <cstdint>

namespace nano_nccl::dev {

constexpr int kMaxBlocks = 160;                       // >= SM count of a B200 (148)
constexpr std::size_t kHalfBytes = 1u << 20;          // staging per block per half
constexpr std::size_t kBlockStageBytes = 2 * kHalfBytes;
constexpr std::size_t kPadBytes = 64 * 1024;          // signal pads (+ room for fused-GEMM flags)
constexpr std::size_t kPadWordsPerBlock = kMaxRanks;
constexpr std::size_t kGemmFlagOffsetBytes = 16 * 1024;  // second pad area inside kPadBytes
constexpr std::size_t kArenaBytes = kPadBytes + kMaxBlocks * kBlockStageBytes;
// Staging of the flag-in-data (LL) kernels: two halves of kLLHalfBytes per block index, in a segment of its own.
constexpr std::size_t kLLHalfBytes = 128 * 1024;
constexpr std::size_t kLLArenaBytes = kMaxBlocks * 2 * kLLHalfBytes;
constexpr int kCollectiveThreads = 512;

// Error codes a kernel may leave in status[0].
enum StatusCode : std::uint32_t {
    kStatusOk = 0,
    kStatusWaitTimeout = 1,   // a bounded wait on a peer ran out
    kStatusAborted = 2,       // host raised the abort word
    kStatusBadArgument = 3,   // debug bounds check tripped
};

// Per-block persistent counters kept in this rank's own memory between launches.
struct BlockState {
    std::uint32_t epoch;  // value of the last barrier this block completed
    std::uint32_t seq;    // launches this block took part in (staging half = seq & 1)
    std::uint32_t epoch_b;  // second signal counter of the pipelined kernels (kernels/pipelined.cuh)
};

struct CommDev {
    int rank;
    int nranks;
    std::uint32_t* pad[kMaxRanks];   // signal pads of every rank (pad[rank] is local)
    char* stage[kMaxRanks];          // staging base of every rank
    char* stage_mc;                  // multicast alias of the staging base, or nullptr
    BlockState* state;               // local, kMaxBlocks entries
    volatile std::uint32_t* status;  // host-mapped: code, peer, phase, block
    const volatile std::uint32_t* abort_flag;  // host-mapped, set by the host to cancel waits
    unsigned long long timeout_ns;
};

// Staging of the flag-in-data (LL) kernels (kernels/ll_collectives.cuh).  The flagged words live in a region
// of their own (a separate symmetric segment), never touched by the other kernels: a stale word left there
// always carries an OLD sequence number in its flag positions, whereas ordinary staging holds arbitrary user
// data that could imitate a flag.
struct LLDev {
    char* stage[kMaxRanks];  // every rank's region (stage[rank] is local)
    char* stage_mc;          // multicast alias, or nullptr
};

}  // namespace nano_nccl::dev
