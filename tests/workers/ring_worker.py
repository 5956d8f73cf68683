"""One rank of the Ring / Simple fallback test: the same AR / RS / AG matrix through the ring
kernels over the requested transport (p2p regions, host shared memory, or socket proxies)."""
import os
import sys

import torch

from nano_nccl_b200 import Communicator

sys.path.insert(0, os.path.dirname(__file__))
import collective_worker  # noqa: E402
from collective_worker import DTYPES, OPS, check, inputs, reference  # noqa: E402

# every ring hop rounds the partial result to the element type: allow one rounding per hop
for _k in collective_worker.TOL:
    collective_worker.TOL[_k] *= max(1, int(os.environ["WORLD_SIZE"]) - 1)

RANK = int(os.environ["RANK"])
SIZE = int(os.environ["WORLD_SIZE"])
PORT = int(os.environ["NANO_TEST_PORT"])
TRANSPORT = sys.argv[1]


def main():
    torch.cuda.set_device(RANK % torch.cuda.device_count())
    dev = torch.device("cuda", torch.cuda.current_device())
    comm = Communicator.from_tcp("127.0.0.1", PORT, RANK, SIZE, device=dev.index, transport=TRANSPORT, algo="ring",
                                 wait_timeout_us=15_000_000)
    want_transport = "p2p" if TRANSPORT in ("auto", "p2p") else TRANSPORT
    assert comm.transport == want_transport, comm.transport
    for r in range(SIZE):
        assert comm.edge_transport(r) == want_transport and not comm.edge_uses_gdr(r)
    seed = 0
    # 16385: odd, more than one slice, less than a slot; 3 Mi + 3: several FIFO generations per channel
    for count in (1, 16385, 3 * 1024 * 1024 + 3):
        for dtype in DTYPES:
            for op in OPS if count != 3 * 1024 * 1024 + 3 else ["sum", "max"]:
                seed += 1
                xs = inputs(count, dtype, seed)
                recv = torch.full((count,), -9137.25, dtype=dtype, device=dev)
                comm.all_reduce(xs[RANK].to(dev), recv, op)
                assert comm.last_algo == "ring"
                # ring hops round partial sums to the element type: allow SIZE roundings
                check(f"ring all_reduce {TRANSPORT} {dtype} {op} n={count}", recv, reference(xs, op), dtype)
                xs = inputs(count * SIZE, dtype, seed + 3)
                out = torch.full((count,), -9137.25, dtype=dtype, device=dev)
                comm.reduce_scatter(xs[RANK].to(dev), out, op)
                check(f"ring reduce_scatter {TRANSPORT} {dtype} {op} n={count}", out,
                      reference(xs, op)[RANK * count:(RANK + 1) * count], dtype)
            xs = inputs(count, dtype, seed + 11)
            allg = torch.full((count * SIZE,), -9137.25, dtype=dtype, device=dev)
            comm.all_gather(xs[RANK].to(dev), allg)
            torch.cuda.synchronize()
            assert torch.equal(allg.cpu(), torch.cat(xs)), f"ring all_gather {TRANSPORT} {dtype} n={count}"
    torch.cuda.synchronize()
    comm.check_async_error()
    assert comm.stats()["ring"] > 0
    # barrier() on a ring transport really waits for the last rank: rank 1 arrives half a second late
    import time

    comm.barrier()
    torch.cuda.synchronize()
    if RANK == 1:
        time.sleep(0.5)
    t0 = time.perf_counter()
    comm.barrier()
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    if RANK != 1:
        assert waited > 0.3, f"barrier returned after {waited:.3f} s although rank 1 was 0.5 s late"
    # A peer that finishes first closes its connections, which a proxy reports as a failure (a
    # closed peer cannot be told from a dead one): agree that everybody is done before leaving.
    done = torch.ones(8, device=dev)
    out = torch.empty(8, device=dev)
    comm.all_reduce(done, out, "sum")
    torch.cuda.synchronize()
    assert float(out[0]) == SIZE
    print(f"[rank {RANK}] ring {TRANSPORT} ok")
    comm.destroy()


if __name__ == "__main__":
    main()
