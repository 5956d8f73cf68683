"""Builds the UNMODIFIED reference library and its two benchmark binaries for comparison runs.

The reference (a CMake project) needs MPI and libnuma, neither of which exists on the target image.
This script compiles the reference's own source files straight from the reference tree with nvcc for
`-arch=sm_100` (the reference's build accepts numeric architectures only), against two stand-ins:
`baseline/shims/numa.h` (reports "no NUMA") and this repository's minimal MPI (`mpi.h` plus
`libminimpi.so`, built here from csrc/minimpi and the bootstrap sources).  Rank and channel counts
are compile-time constants of the reference, so one pair of binaries is built per (ranks, channels).

Products go to baseline/_ref/ (git-ignored):  ref_all_reduce_bench_n<N>_c<C>, ref_collective_bench_n<N>_c<C>,
libminimpi.so.

    python -m baseline.build_reference [--reference <reference tree>] --ranks 2,4,8 --channels 1,2,3,4
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
OUT = ROOT / "baseline" / "_ref"
CSRC = ROOT / "nano_nccl_b200" / "csrc"
CUDA = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))

LIB_SOURCES = [
    "src/c_api.cc", "src/core/buffer.cu", "src/core/numa.cu", "src/transport/p2p/p2p_fifo.cu",
    "src/transport/p2p/p2p_step_counters.cu", "src/transport/p2p/p2p_topology.cu",
    "src/transport/socket/socket_endpoint.cc", "src/transport/socket/socket_proxy.cc",
    "src/collective/all_reduce/topology.cc", "src/collective/all_reduce/communicator.cu", "src/benchmark.cc",
    "src/collective/all_reduce/mpi_communicator.cc", "src/transport/p2p/mpi_p2p.cc", "src/transport/shm/mpi_shm.cc",
]
BENCHES = {"ref_all_reduce_bench": "benchmarks/all_reduce_bench.cu", "ref_collective_bench": "benchmarks/collective_bench.cu"}


def run(cmd):
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError("failed: " + " ".join(map(str, cmd)) + "\n" + p.stdout[-3000:] + p.stderr[-6000:])


def build_minimpi() -> Path:
    OUT.mkdir(parents=True, exist_ok=True)
    lib = OUT / "libminimpi.so"
    srcs = [CSRC / "minimpi" / "minimpi.cc", CSRC / "bootstrap" / "bootstrap.cc", CSRC / "bootstrap" / "tcp_bootstrap.cc",
            CSRC / "core" / "env.cc"]
    run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-I", str(CSRC), "-I", str(CSRC / "include"),
         "-I", str(CSRC / "minimpi"), "-I", str(CUDA / "include")] + [str(s) for s in srcs] + ["-o", str(lib)])
    return lib


def build_variant(ref: Path, nranks: int, channels: int, jobs: int) -> list[Path]:
    objdir = OUT / f"obj_n{nranks}_c{channels}"
    objdir.mkdir(parents=True, exist_ok=True)
    flags = ["-arch=sm_100", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", f"-DNANO_NCCL_NRANKS={nranks}",
             f"-DNANO_NCCL_NCHANNELS={channels}", "-DNANO_NCCL_BLOCK_THREADS=288", "-DNANO_NCCL_FLOAT4_UNROLL=8",
             "-DNANO_NCCL_FIFO_BUFF_BYTES=33554432", "-DNANO_NCCL_ENABLE_MPI=1", "-DOMPI_SKIP_MPICXX",
             "-I", str(ref / "include"), "-I", str(ref / "src"), "-I", str(ROOT / "baseline" / "shims"),
             "-I", str(CSRC / "minimpi"), "-x", "cu"]

    def compile_one(rel: str) -> Path:
        obj = objdir / (rel.replace("/", "_") + ".o")
        run([str(CUDA / "bin" / "nvcc")] + flags + ["-c", str(ref / rel), "-o", str(obj)])
        return obj

    with ThreadPoolExecutor(max_workers=jobs) as pool:
        lib_objs = list(pool.map(compile_one, LIB_SOURCES))
        bench_objs = dict(zip(BENCHES, pool.map(compile_one, BENCHES.values())))
    outs = []
    for name, obj in bench_objs.items():
        exe = OUT / f"{name}_n{nranks}_c{channels}"
        run([str(CUDA / "bin" / "nvcc"), "-arch=sm_100", "-o", str(exe), str(obj)] + [str(o) for o in lib_objs] +
            ["-L", str(OUT), "-lminimpi", "-L", str(CUDA / "lib64" / "stubs"), "-lnvidia-ml", "-lpthread", "-lrt", "-ldl",
             "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"])
        outs.append(exe)
    return outs


def default_reference_path() -> str:
    """`reference_path` of BASELINE.json at the repository root, or the NANO_NCCL_REFERENCE variable."""
    env = os.environ.get("NANO_NCCL_REFERENCE", "")
    if env:
        return env
    try:
        return str(json.loads((ROOT / "BASELINE.json").read_text())["reference_path"])
    except (OSError, KeyError, ValueError):
        return ""


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=default_reference_path(),
                    help="the reference tree (default: reference_path of BASELINE.json)")
    ap.add_argument("--ranks", default="2,4,8")
    ap.add_argument("--channels", default="1,2,3,4")
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    args = ap.parse_args()
    ref = Path(args.reference)
    if not (ref / "src" / "c_api.cc").exists():
        sys.exit(f"{ref} is not the reference tree")
    print("minimpi:", build_minimpi())
    for n in (int(x) for x in args.ranks.split(",")):
        for c in (int(x) for x in args.channels.split(",")):
            for exe in build_variant(ref, n, c, args.jobs):
                print("built", exe)


if __name__ == "__main__":
    main()
