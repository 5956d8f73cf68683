"""Communicator life-cycle cases that mirror the reference's integration tests, one rank per GPU:

    faults      transport fault injection (reference tests/mpi_transport_faults.cc:15-53): with
                NANO_NCCL_TEST_TRANSPORT_FAILURE set, creating a communicator fails on EVERY rank with
                an "injected" error, and a fresh communicator can be created afterwards.
    same_device both ranks pick CUDA device 0 (reference tests/mpi_device_selection.cc): every rank gets
                an error that says the ranks selected the same CUDA device.
    teardown    two communicators at once, the first destroyed, a replacement created and destroyed
                (reference tests/mpi_c_api.cu "partial teardown"); 1 Mi-element AllReduce / ReduceScatter /
                AllGather in float and bf16 on the survivor.

All failures are produced on the host; no kernel is launched on the failing paths.  The cases join the
GPU suite once they have passed on a multi-GPU box.
"""
import os
import sys

import torch

from nano_nccl_b200 import Communicator

sys.path.insert(0, os.path.dirname(__file__))
from collective_worker import check, inputs, reference  # noqa: E402

RANK, SIZE = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
PORT = int(os.environ["NANO_TEST_PORT"])
MODE = sys.argv[1]


def make(port_offset, **kw):
    # the device is named explicitly: a failed creation may leave another device current in this process
    return Communicator.from_tcp("127.0.0.1", PORT + port_offset, RANK, SIZE, device=kw.pop("device", RANK % torch.cuda.device_count()),
                                 wait_timeout_us=15_000_000, **kw)


def smoke(comm, count=1 << 20):
    dev = torch.device("cuda", torch.cuda.current_device())
    for dtype in (torch.float32, torch.bfloat16):
        xs = inputs(count, dtype, 3)
        out = torch.empty(count, dtype=dtype, device=dev)
        comm.all_reduce(xs[RANK].to(dev), out, "sum")
        check("all_reduce", out, reference(xs, "sum"), dtype)
        xs = inputs(count * SIZE, dtype, 4)
        part = torch.empty(count, dtype=dtype, device=dev)
        comm.reduce_scatter(xs[RANK].to(dev), part, "sum")
        check("reduce_scatter", part, reference(xs, "sum")[RANK * count:(RANK + 1) * count], dtype)
        xs = inputs(count, dtype, 5)
        full = torch.empty(count * SIZE, dtype=dtype, device=dev)
        comm.all_gather(xs[RANK].to(dev), full)
        torch.cuda.synchronize()
        assert torch.equal(full.cpu(), torch.cat(xs))
    comm.check_async_error()


def faults():
    offset = 0
    for point, transport in (("shm_allocation", "shm"), ("shm_registration", "shm"), ("p2p_allocation", "p2p"), ("p2p_open", "p2p")):
        os.environ["NANO_NCCL_TEST_TRANSPORT_FAILURE"] = point
        try:
            make(offset, transport=transport, algo="ring")
        except Exception as e:  # every rank, not only the one that injected
            assert "injected" in str(e), (point, str(e))
        else:
            raise AssertionError(f"[rank {RANK}] {point}: communicator creation succeeded")
        del os.environ["NANO_NCCL_TEST_TRANSPORT_FAILURE"]
        offset += 1
        comm = make(offset, transport=transport, algo="ring")   # cleanup was complete: a fresh one works
        smoke(comm, 16385)
        comm.destroy()
        offset += 1


def same_device():
    try:
        make(0, device=0)
    except Exception as e:
        assert "same CUDA device" in str(e), str(e)
    else:
        raise AssertionError(f"[rank {RANK}] two ranks on device 0 were accepted")
    torch.cuda.set_device(RANK % torch.cuda.device_count())
    comm = make(1)   # with distinct devices everything is fine afterwards
    smoke(comm, 4096)
    comm.destroy()


def teardown():
    first, second = make(0), make(1)
    import ctypes as C

    from nano_nccl_b200 import _native as N

    channels = C.c_int(0)
    N.load_library().nano_nccl_mpi_channel_count.argtypes = [C.POINTER(C.c_int)]
    assert N.load_library().nano_nccl_mpi_channel_count(C.byref(channels)) == 0 and channels.value == 4
    for r in range(SIZE):
        assert second.edge_transport(r) == "p2p"
    try:
        second.edge_transport(SIZE)
    except ValueError as e:
        assert "edge" in str(e)
    else:
        raise AssertionError("invalid edge accepted")
    first.destroy()
    replacement = make(2)
    smoke(replacement, 4096)
    replacement.destroy()
    smoke(second)
    second.destroy()


def main():
    torch.cuda.set_device(RANK % torch.cuda.device_count())
    {"faults": faults, "same_device": same_device, "teardown": teardown}[MODE]()
    print(f"[rank {RANK}] {MODE} ok")


if __name__ == "__main__":
    main()
