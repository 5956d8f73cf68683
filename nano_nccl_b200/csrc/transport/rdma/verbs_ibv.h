// Internal face of the libibverbs provider: the run-time binding of the library and a constructor that takes
// the function table and the device choice explicitly, so that a test can drive the provider against a fake
// table and check the attributes it programs (queue pair creation, INIT -> RTR -> RTS) without an HCA.
#pragma once

#include "transport/rdma/ibverbs_abi.h"
#include "transport/rdma/rdma_endpoint.h"
#include "transport/rdma/verbs.h"

#include <memory>
#include <string>

namespace nano_nccl::rdma {

// dlopen("libibverbs.so.1") and every entry point of IbvApi, once per process; nullptr (with `why`) when the
// library or one of the required entry points is missing.  reg_dmabuf_mr is optional.
const IbvApi* load_ibverbs(std::string* why);

// Opens `choice.hca` through `api`.  Throws std::runtime_error with the failing step.
std::shared_ptr<VerbsDevice> open_ibverbs_device_with(const IbvApi& api, const HcaChoice& choice);

}  // namespace nano_nccl::rdma
