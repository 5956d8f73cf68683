"""A communicator whose drain fails during destruction (injected on the host: NANO_NCCL_TEST_TEARDOWN_FAILURE=1
makes the destructor treat its own successful device synchronisation as failed; no GPU error is produced).

    quarantine  default policy: a line on stderr, the memory stays mapped, the process goes on and a fresh
                communicator works
    abort       NANO_NCCL_TEARDOWN=abort: the process ends (the reference's fail-stop behaviour,
                src/collective/all_reduce/communicator.cu:108-119)
"""
import os
import sys

import torch

from nano_nccl_b200 import Communicator

PORT = int(os.environ["NANO_TEST_PORT"])
MODE = sys.argv[1]
torch.cuda.set_device(0)
x = torch.randn(4096, device="cuda")
y = torch.empty_like(x)
comm = Communicator.from_tcp("127.0.0.1", PORT, 0, 1, device=0)
comm.all_reduce(x, y, "sum")
torch.cuda.synchronize()
os.environ["NANO_NCCL_TEST_TEARDOWN_FAILURE"] = "1"
if MODE == "abort":
    os.environ["NANO_NCCL_TEARDOWN"] = "abort"
print("destroying", flush=True)
comm.destroy()          # abort mode never returns
del os.environ["NANO_NCCL_TEST_TEARDOWN_FAILURE"]
again = Communicator.from_tcp("127.0.0.1", PORT + 1, 0, 1, device=0)
again.all_reduce(x, y, "sum")
torch.cuda.synchronize()
assert torch.equal(x, y)
again.destroy()
print("teardown policy ok")
