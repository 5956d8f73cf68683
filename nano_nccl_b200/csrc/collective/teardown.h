// What a communicator does when draining its own GPU work fails during destruction.
//
// The reference ends the process (std::terminate) when CUDA fails while it releases its lifetime tracking
// (src/collective/all_reduce/communicator.cu:108-119, 1303-1321): after such a failure it cannot know whether a
// kernel still uses the memory it is about to free.  This library lives inside training frameworks, where ending
// the process loses the caller's own error report, so the default is to QUARANTINE instead: say what failed on
// stderr and leave every mapping, staging buffer and peer mapping of the communicator in place (a deliberate
// leak: nothing a surviving kernel or a peer can still touch is unmapped).  NANO_NCCL_TEARDOWN=abort restores
// the reference's fail-stop behaviour; NANO_NCCL_TEARDOWN=quarantine (or unset) is the default.
#pragma once

#include <stdexcept>
#include <string>

namespace nano_nccl {

enum class TeardownAction { Release, Quarantine, Abort };

// `policy`: the value of NANO_NCCL_TEARDOWN ("" when unset).  Throws std::invalid_argument for other values.
inline TeardownAction decide_teardown(bool drain_failed, const std::string& policy) {
    if (!(policy.empty() || policy == "quarantine" || policy == "abort")) {
        throw std::invalid_argument("NANO_NCCL_TEARDOWN must be unset, 'quarantine' or 'abort', got '" + policy + "'");
    }
    if (!drain_failed) return TeardownAction::Release;
    return policy == "abort" ? TeardownAction::Abort : TeardownAction::Quarantine;
}

}  // namespace nano_nccl
