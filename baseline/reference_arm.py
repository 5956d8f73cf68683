"""The reference arm of bench.py: runs the unmodified reference library, as far as it can go.

The reference (a C++/CUDA/CMake project) has no Python packaging, so `pip install` into baseline/_ref
cannot succeed, and it has no model, no torch binding and no one-rank mode, so it cannot produce a
training-throughput number at any rank count: for that value the arm reports `unavailable`.

What the reference does produce is the metric its own documentation publishes: the AllReduce /
ReduceScatter / AllGather tables of its two benchmark programs.  baseline/build_reference.py compiles the
reference's sources unmodified (stand-ins only for libnuma and MPI, which the image lacks) into
baseline/_ref/ref_{all_reduce,collective}_bench_n<N>_c<C>; at 2, 4 or 8 GPUs this arm runs them with the
reference's stock arguments and loop (`-b 262144 -e 67108864 -f 4 -w 5 -n 20`; host wall clock around
enqueue + wait, mean of n, max over ranks, every element verified: reference
benchmarks/all_reduce_bench.cu:142-173, benchmarks/collective_bench.cu:195-197) for every channel count
that is built, and reports the parsed tables under `collectives`, the same (collective, dtype, bytes)
grid that bench.py's own arm reports.
"""
from __future__ import annotations

import math
import subprocess
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
REF_DIR = ROOT / "baseline" / "_ref"
MPIRUN = ROOT / "nano_nccl_b200" / "lib" / "nano_nccl_mpirun"
SIZES = (262144, 67108864, 4)  # -b, -e, -f
DTYPES = ("float", "fp16", "bf16")
COLLECTIVES = ("all_reduce", "reduce_scatter", "all_gather")
CHANNEL_ORDER = (4, 2, 1, 3)  # most important first, in case the time budget runs out

WHY_NO_TRAINING_VALUE = (
    "the reference is a C++/CUDA collective library without a model, a training step, a torch binding or a one-rank "
    "mode, so it cannot produce tokens/s (pip install of its tree fails: no setup.py / pyproject.toml); its own "
    "benchmark programs, built unmodified for sm_100, are run instead and reported under 'collectives'")


def parse_reference_table(text: str) -> list[dict]:
    """Rows of the reference's programs: algo dtype redop transport size count time_us algbw busbw wrong max_abs."""
    rows = []
    for line in text.splitlines():
        parts = line.split()
        if len(parts) == 11 and not line.startswith("#") and parts[4].isdigit():
            try:
                rows.append({"dtype": parts[1], "transport": parts[3], "bytes": int(parts[4]), "time_us": float(parts[6]),
                             "algbw_gbs": float(parts[7]), "busbw_gbs": float(parts[8]), "wrong": int(parts[9])})
            except ValueError:
                continue
    return rows


def _geomean(values) -> float | None:
    values = [v for v in values if v and v > 0]
    return round(math.exp(sum(math.log(v) for v in values) / len(values)), 3) if values else None


def run_one(nranks: int, channels: int, collective: str, dtype: str, timeout_s: int) -> tuple[list[dict], str]:
    common = ["--dtype", dtype, "-b", str(SIZES[0]), "-e", str(SIZES[1]), "-f", str(SIZES[2]), "-w", "5", "-n", "20"]
    if collective == "all_reduce":
        exe, args = REF_DIR / f"ref_all_reduce_bench_n{nranks}_c{channels}", ["--redop", "sum"] + common
    elif collective == "reduce_scatter":
        exe, args = REF_DIR / f"ref_collective_bench_n{nranks}_c{channels}", ["--collective", "reducescatter", "--redop", "sum"] + common
    else:  # the reference rejects a reduction operator for AllGather
        exe, args = REF_DIR / f"ref_collective_bench_n{nranks}_c{channels}", ["--collective", "allgather"] + common
    if not exe.exists():
        return [], f"{exe.name} is not built (python -m baseline.build_reference --ranks {nranks} --channels {channels})"
    cmd = [str(MPIRUN), "-np", str(nranks), "--timeout", str(timeout_s), str(exe)] + args
    try:
        p = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s + 20)
    except subprocess.TimeoutExpired:
        return [], "launcher timeout"
    rows = parse_reference_table(p.stdout)
    # bus bandwidth by the reference's own conventions; its AllReduce program prints it, recomputed here for both
    factor = (2.0 if collective == "all_reduce" else 1.0) * (nranks - 1) / nranks
    for r in rows:
        r["collective"] = collective
        r["busbw_gbs"] = round(r["bytes"] / r["time_us"] / 1e3 * factor, 3) if r["time_us"] > 0 else 0.0
    note = ""
    if p.returncode != 0 or not rows:
        note = f"exit {p.returncode}: " + " | ".join((p.stdout + p.stderr).strip().splitlines()[-2:])[:300]
    return rows, note


def reference_collectives(nranks: int, budget_s: float = 240.0, timeout_s: int = 90) -> dict:
    """Every built channel count x collective x dtype, most important first, within a time budget."""
    t0 = time.time()
    per_channel: dict[str, dict] = {}
    for channels in CHANNEL_ORDER:
        cells, notes = [], []
        for collective in COLLECTIVES:
            for dtype in DTYPES:
                if time.time() - t0 > budget_s:
                    notes.append(f"{collective}/{dtype}: skipped, time budget of {budget_s:.0f} s used up")
                    continue
                rows, note = run_one(nranks, channels, collective, dtype, timeout_s)
                cells += rows
                if note:
                    notes.append(f"{collective}/{dtype}: {note}")
        entry = {"geomean_busbw_gbs": _geomean(c["busbw_gbs"] for c in cells),
                 "wrong_elements": sum(c["wrong"] for c in cells), "cells": cells}
        if notes:
            entry["notes"] = notes
        per_channel[str(channels)] = entry
    best = max((e["geomean_busbw_gbs"] or 0.0 for e in per_channel.values()), default=0.0)
    return {"timing": "the reference's stock loop: host wall clock around enqueue + wait, mean of 20 after 5 warm-ups, "
                      "max over ranks; op sum; bytes = AllReduce message or the whole N-chunk buffer",
            "nranks": nranks, "best_geomean_busbw_gbs": best or None, "elapsed_s": round(time.time() - t0, 1),
            "channels": per_channel}


def run_reference(gpus: int, steps: int, warmup: int, budget_s: float = 240.0) -> dict:
    out = {"impl": "reference", "unavailable": WHY_NO_TRAINING_VALUE, "n_gpus": gpus, "steps": steps, "warmup": warmup,
           "metric": "DP training tokens/s, GPT-2-medium, BF16 (collectives: AllReduce avg of 25 MB buckets)", "value": None}
    if gpus in (2, 4, 8) and MPIRUN.exists():
        out["collectives"] = reference_collectives(gpus, budget_s)
    elif gpus >= 2:
        out["collectives"] = {"unavailable": f"the reference fixes its rank count at build time; built: 2, 4, 8, asked: {gpus}"}
    return out
