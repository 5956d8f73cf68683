"""The headline collective grid: AllReduce / ReduceScatter / AllGather x {float, fp16, bf16} x message
sizes 256 KiB .. 64 MiB (x4), sum, tuner defaults, ordinary (unregistered) buffers, for this library and
for NCCL in the same process.  Per cell: 5 warm-up and 20 timed iterations, each timed on the device with
CUDA events after an L2 flush and a device-side alignment of the ranks; p50 per rank, MAX over ranks.

Bus bandwidth follows the reference (src/benchmark.cc:22-29, benchmarks/collective_bench.cu:195-197):
AllReduce S/t * 2(N-1)/N; ReduceScatter / AllGather S_total/t * (N-1)/N, where S_total is the whole
N-chunk buffer.  `bytes` is the AllReduce message or S_total, which is also what `-b` / `-e` mean to the
reference's benchmark programs, so cells of both line up by (collective, dtype, bytes).

`bench.py` calls :func:`collective_grid` after its training measurement; `native_table` runs this library's
native benchmark programs (the reference's host-timed loop) for the like-for-like table.
"""
from __future__ import annotations

import math
import subprocess
import time
from pathlib import Path

SIZES = [256 * 1024 * 4 ** i for i in range(5)]  # 256 KiB .. 64 MiB
DTYPES = ("float", "fp16", "bf16")
COLLECTIVES = ("all_reduce", "reduce_scatter", "all_gather")
LIB = Path(__file__).resolve().parents[1] / "lib"


def busbw_factor(collective: str, world: int) -> float:
    return (2.0 if collective == "all_reduce" else 1.0) * (world - 1) / world


def geomean(values) -> float | None:
    values = [v for v in values if v and v > 0]
    if not values:
        return None
    return math.exp(sum(math.log(v) for v in values) / len(values))


def summarize(cells: list[dict]) -> dict:
    """Geomeans over the cells; `vs_nccl` is NCCL time / this library's time over matched cells."""
    out = {"geomean_busbw_gbs": geomean(c["busbw_gbs"] for c in cells if c["impl"] == "nano")}
    nccl = {(c["collective"], c["dtype"], c["bytes"]): c for c in cells if c["impl"] == "nccl"}
    ratios, slower = [], []
    for c in cells:
        if c["impl"] != "nano":
            continue
        key = (c["collective"], c["dtype"], c["bytes"])
        if key in nccl and c["p50_us"] > 0:
            r = nccl[key]["p50_us"] / c["p50_us"]
            ratios.append(r)
            if r < 1.0:
                slower.append({"collective": key[0], "dtype": key[1], "bytes": key[2], "ratio": round(r, 3)})
    if ratios:
        out["nccl_geomean_busbw_gbs"] = geomean(c["busbw_gbs"] for c in nccl.values())
        out["geomean_nccl_time_over_nano_time"] = round(geomean(ratios), 4)
        out["cells_faster_than_nccl"] = sum(1 for r in ratios if r >= 1.0)
        out["cells_compared"] = len(ratios)
        out["cells_slower_than_nccl"] = slower
    for k in ("geomean_busbw_gbs", "nccl_geomean_busbw_gbs"):
        if out.get(k) is not None:
            out[k] = round(out[k], 2)
    return out


def collective_grid(comm, world: int, *, dtypes=DTYPES, sizes=SIZES, collectives=COLLECTIVES, iters: int = 20,
                    warmup: int = 5, with_nccl: bool = True) -> dict:
    """Runs the grid on an existing communicator (all ranks call it); returns {"cells": [...], summary...}."""
    import torch
    import torch.distributed as dist

    from nano_nccl_b200.utils.timing import L2Flusher, max_over_ranks, p50, time_iterations

    dt = {"float": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}
    flush = L2Flusher()
    align = torch.zeros(1, device="cuda")

    def aligned():
        dist.all_reduce(align)  # device-side: every rank's timed region starts together

    comm.set_algo("auto")
    comm.set_grid_override(0)
    cells = []
    launches = 0
    for coll in collectives:
        factor = busbw_factor(coll, world)
        for dname in dtypes:
            dtype = dt[dname]
            esz = torch.empty((), dtype=dtype).element_size()
            for nbytes in sizes:
                if coll == "all_reduce":
                    count = nbytes // esz
                    send = torch.rand(count, device="cuda").mul_(2).sub_(1).to(dtype)
                    recv = torch.empty_like(send)
                    total = nbytes
                    fns = {"nano": lambda: comm.all_reduce(send, recv, "sum"),
                           "nccl": lambda: dist.all_reduce(recv)}  # in place: NCCL's best case
                else:
                    count = nbytes // esz // world
                    big = torch.rand(count * world, device="cuda").mul_(2).sub_(1).to(dtype)
                    small = torch.empty(count, dtype=dtype, device="cuda")
                    total = count * world * esz
                    if coll == "reduce_scatter":
                        fns = {"nano": lambda: comm.reduce_scatter(big, small, "sum"),
                               "nccl": lambda: dist.reduce_scatter_tensor(small, big)}
                    else:
                        fns = {"nano": lambda: comm.all_gather(small, big),
                               "nccl": lambda: dist.all_gather_into_tensor(big, small)}
                for impl in ("nano", "nccl") if with_nccl else ("nano",):
                    times = time_iterations(fns[impl], iters, warmup, flush=flush, pre=aligned)
                    t50 = max_over_ranks(p50(times))
                    if impl == "nano":
                        launches += iters + warmup
                    cells.append({"collective": coll, "dtype": dname, "bytes": total, "impl": impl,
                                  "algo": comm.last_algo if impl == "nano" else "nccl",
                                  "p50_us": round(t50, 2), "busbw_gbs": round(total / t50 / 1e3 * factor, 2)})
    comm.check_async_error()
    out = {"timing": f"device (CUDA events), p50 of {iters} after {warmup} warm-ups, max over ranks, L2 flushed, op sum, "
                     "ordinary buffers, tuner defaults", "nranks": world, "nano_kernel_launches": launches}
    out.update(summarize(cells))
    out["cells"] = cells
    return out


def parse_nano_bench(text: str) -> list[dict]:
    """Rows of this library's native benchmark programs:
    collective dtype op algo bytes count host_us dev_p50us dev_avgus algbw busbw wrong max_abs."""
    rows = []
    for line in text.splitlines():
        parts = line.split()
        if len(parts) == 13 and not line.startswith("#") and parts[4].isdigit():
            rows.append({"collective": parts[0], "dtype": parts[1], "bytes": int(parts[4]), "algo": parts[3],
                         "host_us": float(parts[6]), "dev_p50_us": float(parts[7]), "busbw_gbs": float(parts[10]),
                         "wrong": int(parts[11])})
    return rows


def native_table(nranks: int, *, dtypes=DTYPES, budget_s: float = 120.0, timeout_s: int = 60) -> dict:
    """This library's native benchmark programs under the bundled launcher with the arguments the reference's
    programs get (`-b 262144 -e 67108864 -f 4 -w 5 -n 20`): the reference's loop (host wall clock around
    enqueue + wait, mean of n, max over ranks, every element verified).  One process; call from one rank only,
    while no other work runs on the GPUs."""
    mpirun = LIB / "nano_nccl_mpirun"
    t0 = time.time()
    cells, notes = [], []
    for coll in COLLECTIVES:
        exe = LIB / ("nano_nccl_all_reduce_bench" if coll == "all_reduce" else "nano_nccl_collective_bench")
        for dname in dtypes:
            if time.time() - t0 > budget_s:
                notes.append(f"{coll}/{dname}: skipped, time budget of {budget_s:.0f} s used up")
                continue
            args = ["--collective", coll, "--dtype", dname, "-b", str(SIZES[0]), "-e", str(SIZES[-1]), "-f", "4",
                    "-w", "5", "-n", "20"]
            if coll != "all_gather":
                args = ["--redop", "sum"] + args
            cmd = [str(mpirun), "-np", str(nranks), "--timeout", str(timeout_s), str(exe)] + args
            try:
                p = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s + 20)
                rows = parse_nano_bench(p.stdout)
                for r in rows:  # the bandwidth column of the program uses the device time; this table is the host loop
                    r["busbw_gbs"] = round(r["bytes"] / r["host_us"] / 1e3 * busbw_factor(coll, nranks), 2) if r["host_us"] > 0 else 0.0
                if p.returncode != 0 or not rows:
                    notes.append(f"{coll}/{dname}: exit {p.returncode}: " + " | ".join((p.stdout + p.stderr).strip().splitlines()[-2:])[:300])
                cells += rows
            except subprocess.TimeoutExpired:
                notes.append(f"{coll}/{dname}: launcher timeout")
    out = {"timing": "host wall clock around enqueue + wait, mean of 20 after 5 warm-ups, max over ranks "
                     "(the loop of the reference's benchmark programs)",
           "geomean_busbw_gbs": geomean(c["busbw_gbs"] for c in cells), "wrong_elements": sum(c["wrong"] for c in cells),
           "cells": cells}
    if out["geomean_busbw_gbs"] is not None:
        out["geomean_busbw_gbs"] = round(out["geomean_busbw_gbs"], 2)
    if notes:
        out["notes"] = notes
    return out
