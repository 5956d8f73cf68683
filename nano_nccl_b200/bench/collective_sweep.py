"""Bus-bandwidth and latency sweep of AllReduce / ReduceScatter / AllGather against NCCL.

Launch with torchrun (one process per GPU).  Per cell: 5 warm-up and 20 timed iterations, each
timed on the device with CUDA events after an L2 flush and a device-side rank alignment; p50 per
rank, then the MAX over ranks.  Bus bandwidth follows the reference's conventions
(src/benchmark.cc:22-29 and benchmarks/collective_bench.cu:195-197):
AllReduce S/t * 2(N-1)/N; ReduceScatter / AllGather S_total/t * (N-1)/N.

Usage: torchrun --nproc-per-node N -m nano_nccl_b200.bench.collective_sweep [--out file.jsonl]

`--variants "default;NANO_NCCL_PIPE_MIN_BYTES=0;NANO_NCCL_LL_MAX_BYTES=1048576"` repeats the sweep of this library
once per environment variant in the same process (the switches are read when a communicator is created, so every
variant gets a communicator of its own); NCCL is timed once.  Rows carry a "variant" field.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch
import torch.distributed as dist

from nano_nccl_b200.communicator import Communicator
from nano_nccl_b200.utils.timing import L2Flusher, max_over_ranks, p50, time_iterations

DT = {"float": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def sizes(lo: int, hi: int, factor: int, extra: list[int]) -> list[int]:
    out, s = [], lo
    while s <= hi:
        out.append(s)
        s *= factor
    return out + [e for e in extra if e not in out]


def apply_variant(variant: str) -> dict:
    """Sets the variant's environment variables; returns what to restore."""
    saved = {}
    if variant != "default":
        for pair in variant.split(","):
            k, v = pair.split("=", 1)
            saved[k] = os.environ.get(k)
            os.environ[k] = v
    return saved


def restore_env(saved: dict) -> None:
    for k, v in saved.items():
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--collectives", default="all_reduce,reduce_scatter,all_gather")
    ap.add_argument("--dtypes", default="float,bf16")
    ap.add_argument("--ops", default="sum")
    ap.add_argument("--min-bytes", type=int, default=256 * 1024)
    ap.add_argument("--max-bytes", type=int, default=64 * 1024 * 1024)
    ap.add_argument("--factor", type=int, default=4)
    ap.add_argument("--extra-bytes", default="")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--algos", default="auto", help="comma list: auto,oneshot,twoshot,nvls")
    ap.add_argument("--grids", default="", help="comma list of NANO max CTAs to sweep (tuning)")
    ap.add_argument("--symmetric", action="store_true", help="also time zero-copy symmetric buffers")
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--no-flush", action="store_true", help="tuning only: keep L2 warm between iterations")
    ap.add_argument("--variants", default="",
                    help="';'-separated environment variants (VAR=value[,VAR=value]); 'default' changes nothing")
    ap.add_argument("--out", default="")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    variants = [v.strip() for v in args.variants.split(";") if v.strip()] or ["default"]
    flush = None if args.no_flush else L2Flusher()
    align = torch.zeros(1, device="cuda")
    rows = []
    out_file = None
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        out_file = open(args.out, "w")  # rows are appended as they are measured: a run that is cut short keeps them

    def emit(row):
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
            if out_file is not None:
                out_file.write(json.dumps(row) + "\n")
                out_file.flush()

    def aligned():
        dist.all_reduce(align)  # device-side: every rank's timed region starts together

    extra = [int(x) for x in args.extra_bytes.split(",") if x]

    def sweep(comm, variant: str, with_nccl: bool) -> None:
        for coll in args.collectives.split(","):
            for dname in args.dtypes.split(","):
                dtype = DT[dname]
                esz = torch.empty((), dtype=dtype).element_size()
                for op in (args.ops.split(",") if coll != "all_gather" else ["sum"]):
                    for nbytes in sizes(args.min_bytes, args.max_bytes, args.factor, extra):
                        # nbytes: AllReduce message; RS / AG: the whole N-chunk buffer (per-rank chunk = nbytes / world)
                        if coll == "all_reduce":
                            count = nbytes // esz
                            send = torch.rand(count, device="cuda").mul_(2).sub_(1).to(dtype)
                            recv = torch.empty_like(send)
                            total = nbytes
                            factor = 2 * (world - 1) / world
                        else:
                            count = nbytes // esz // world
                            big = torch.rand(count * world, device="cuda").mul_(2).sub_(1).to(dtype)
                            small = torch.empty(count, dtype=dtype, device="cuda")
                            total = count * world * esz
                            factor = (world - 1) / world
                        impls = []
                        grids = [int(g) for g in args.grids.split(",") if g] or [0]
                        for algo in args.algos.split(","):
                            for grid in grids:
                                impls.append(("nano", algo, grid))
                        if with_nccl:
                            impls.append(("nccl", "default", 0))
                        for impl, algo, grid in impls:
                            if impl == "nano" and coll != "all_reduce" and algo not in ("auto", args.algos.split(",")[0]):
                                continue  # RS / AG have one NVLink algorithm
                            if impl == "nano":
                                comm.set_algo(algo)
                                comm.set_grid_override(grid)
                                if coll == "all_reduce":
                                    fn = lambda: comm.all_reduce(send, recv, op)
                                elif coll == "reduce_scatter":
                                    fn = lambda: comm.reduce_scatter(big, small, op)
                                else:
                                    fn = lambda: comm.all_gather(small, big)
                            else:
                                rop = {"sum": dist.ReduceOp.SUM, "avg": dist.ReduceOp.AVG, "max": dist.ReduceOp.MAX,
                                       "min": dist.ReduceOp.MIN}[op]
                                if coll == "all_reduce":
                                    fn = (lambda: dist.all_reduce(recv, op=rop))  # in place, no copy: NCCL's best case
                                elif coll == "reduce_scatter":
                                    fn = lambda: dist.reduce_scatter_tensor(small, big, op=rop)
                                else:
                                    fn = lambda: dist.all_gather_into_tensor(big, small)
                            times = time_iterations(fn, args.iters, args.warmup, flush=flush, pre=aligned)
                            t50 = max_over_ranks(p50(times))
                            tmin = max_over_ranks(min(times))
                            algbw = total / t50 / 1e3
                            emit({"collective": coll, "dtype": dname, "op": op, "bytes": total, "impl": impl,
                                  "algo": comm.last_algo if impl == "nano" else "nccl", "grid": grid,
                                  "nranks": world, "p50_us": round(t50, 2), "min_us": round(tmin, 2),
                                  "algbw_gbs": round(algbw, 2), "busbw_gbs": round(algbw * factor, 2), "variant": variant})
        comm.check_async_error()

    comm = None
    for vi, variant in enumerate(variants):
        saved = apply_variant(variant)
        if comm is not None:
            comm.destroy()
        comm = Communicator.from_torch_distributed(device=local)
        restore_env(saved)
        sweep(comm, variant, with_nccl=not args.no_nccl and vi == 0)
    if args.symmetric and comm.multicast_available:
        for dname in args.dtypes.split(","):
            dtype = DT[dname]
            esz = torch.empty((), dtype=dtype).element_size()
            for nbytes in sizes(args.min_bytes, args.max_bytes, args.factor, extra):
                count = nbytes // esz
                buf = comm.symmetric_empty(count, dtype)
                buf.copy_(torch.rand(count, device="cuda").to(dtype))
                comm.set_algo("nvls")
                fn = lambda: comm.all_reduce(buf, buf, "avg")
                times = time_iterations(fn, args.iters, args.warmup, flush=flush, pre=aligned)
                t50 = max_over_ranks(p50(times))
                algbw = nbytes / t50 / 1e3
                row = {"collective": "all_reduce", "dtype": dname, "op": "avg", "bytes": nbytes, "impl": "nano",
                       "algo": "nvls_symmetric_inplace", "grid": 0, "nranks": world, "p50_us": round(t50, 2),
                       "min_us": round(max_over_ranks(min(times)), 2), "algbw_gbs": round(algbw, 2),
                       "busbw_gbs": round(algbw * 2 * (world - 1) / world, 2)}
                emit(row)
    if out_file is not None:
        out_file.close()
    if rank == 0:
        # per variant: geomean of NCCL time / this library's time over matched cells (tuner defaults, ordinary buffers)
        nccl = {(r["collective"], r["dtype"], r["op"], r["bytes"]): r for r in rows if r["impl"] == "nccl"}
        for variant in variants:
            ratios, slower = [], 0
            for r in rows:
                key = (r["collective"], r["dtype"], r["op"], r["bytes"])
                if r["impl"] == "nano" and r.get("variant") == variant and "symmetric" not in str(r["algo"]) and key in nccl:
                    ratios.append(nccl[key]["p50_us"] / r["p50_us"])
                    slower += ratios[-1] < 1.0
            if ratios:
                gm = math.exp(sum(math.log(x) for x in ratios) / len(ratios))
                print(json.dumps({"summary": "geomean NCCL time / nano time", "variant": variant, "cells": len(ratios),
                                  "cells_slower_than_nccl": slower, "value": round(gm, 4)}), flush=True)
    comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
