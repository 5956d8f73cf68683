"""Where does the time of a fused GEMM + collective kernel go?  Runs the benchmark problem a few times with the
kernel's diagnostic time line switched on and prints, for this rank, a digest over all CTAs of the last call:

  * span         first kernel entry to last event;
  * mma wait     time the epilogue spent waiting for an accumulator (tag 3 of one tile -> tag 1 of the next):
                 large means the tensor cores (or their operands) are the bottleneck;
  * drain        accumulator complete -> handed back (tag 1 -> tag 3): large means the epilogue (its remote
                 stores) is the bottleneck;
  * peer wait    own tiles: accumulator complete -> partials arrived (tag 1 -> tag 2);
  * block wait   AllGather->GEMM producer waiting for a remote row block (tag 5 -> tag 6);
  * publish      GEMM->ReduceScatter flag publisher inside the release store of a foreign tile's flag
                 (tag 7 -> tag 4): the wait for that tile's remote stores to be acknowledged.

    NANO_NCCL_GEMM_TRACE=1 torchrun --nproc-per-node 8 -m nano_nccl_b200.bench.fused_trace [--op gemm_rs|ag_gemm]

The stamps cost a global-timer read and a store per event, so the traced kernel is a little slower than the
untraced one; the proportions are what matters.
"""
from __future__ import annotations

import argparse
import os
import statistics

import torch
import torch.distributed as dist

from nano_nccl_b200 import Communicator
from nano_nccl_b200.ops.gemm import FusedTensorParallel


def digest(trace: dict) -> dict:
    first = min(ev[0][1] for roles in trace.values() for ev in roles.values())
    last = max(ev[-1][1] for roles in trace.values() for ev in roles.values())
    mma_wait, drain, peer_wait, block_wait, publish, tiles = [], [], [], [], [], []
    for roles in trace.values():
        ep = roles.get("epilogue", [])
        w = d = pw = 0
        ntiles = 0
        prev_back = None
        acc_ready = None
        for tag, t in ep:
            if tag == 0:
                prev_back = t
            elif tag == 1:
                if prev_back is not None:
                    w += t - prev_back
                acc_ready = t
                ntiles += 1
            elif tag == 2 and acc_ready is not None:
                pw += t - acc_ready
            elif tag == 3 and acc_ready is not None:
                d += t - acc_ready
                prev_back = t
        if ntiles:
            mma_wait.append(w)
            drain.append(d)
            peer_wait.append(pw)
            tiles.append(ntiles)
        pr = roles.get("producer", [])
        bw, pb, start = 0, 0, None
        for tag, t in pr:
            if tag in (5, 7):
                start = t
            elif tag == 6 and start is not None:
                bw += t - start
            elif tag == 4 and start is not None:
                pb += t - start
        if pr:
            block_wait.append(bw)
            publish.append(pb)
    med = lambda xs: statistics.median(xs) / 1e3 if xs else 0.0  # noqa: E731
    return {"ctas": len(trace), "span_us": (last - first) / 1e3, "tiles_per_cta": statistics.median(tiles) if tiles else 0,
            "mma_wait_us": med(mma_wait), "drain_us": med(drain), "peer_wait_us": med(peer_wait),
            "publish_us": med(publish), "block_wait_us": med(block_wait), "block_wait_max_us": max(block_wait) / 1e3 if block_wait else 0.0}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemm_rs", choices=["gemm_rs", "ag_gemm"])
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    args = ap.parse_args()
    if os.environ.get("NANO_NCCL_GEMM_TRACE", "") not in ("1", "true", "on"):
        raise SystemExit("set NANO_NCCL_GEMM_TRACE=1")
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl")
    comm = Communicator.from_torch_distributed()
    r, n = comm.rank, comm.size
    m, h, fp = args.tokens, args.hidden, args.ffn // n
    fused = FusedTensorParallel(comm, m * h * 2, m * h * 2)
    torch.manual_seed(r)
    if args.op == "gemm_rs":
        a = torch.randn(m, fp, device="cuda").bfloat16()
        w = (torch.randn(h, fp, device="cuda") * 0.02).bfloat16()
        run = lambda: fused.gemm_rs(a, w)  # noqa: E731
    else:
        x = torch.randn(m // n, h, device="cuda").bfloat16()
        w = (torch.randn(fp, h, device="cuda") * 0.02).bfloat16()
        run = lambda: fused.ag_gemm(x, w)  # noqa: E731
    align = torch.zeros(1, device="cuda")
    for _ in range(4):
        dist.all_reduce(align)
        run()
    torch.cuda.synchronize()
    d = digest(fused.read_trace())
    rows = [None] * n
    dist.all_gather_object(rows, d)
    if r == 0:
        print(f"# {args.op} on {n} GPUs: M={m} hidden={h} ffn/rank={fp}; medians over CTAs, microseconds")
        for i, row in enumerate(rows):
            print(f"rank {i}: " + "  ".join(f"{k}={v:.1f}" if isinstance(v, float) else f"{k}={v}" for k, v in row.items()))
    comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
