"""Small, self-terminating workloads for profiler captures (one GPU, a few hundred MB).

    python -m nano_nccl_b200.bench.profile_cases gemm        # tcgen05 GEMM 16384 x 4096 x 1792, 3 launches
    python -m nano_nccl_b200.bench.profile_cases emu_twoshot # 8 emulated ranks, 32 MiB bf16 two-shot AllReduce
    python -m nano_nccl_b200.bench.profile_cases adamw       # fused AdamW over 64 Mi parameters
    python -m nano_nccl_b200.bench.profile_cases emu_oneshot | emu_reduce_scatter | emu_all_gather   # 8 emulated ranks, 32 MiB
    python -m nano_nccl_b200.bench.profile_cases emu_ll      # 8 emulated ranks, 256 KiB flag-in-data AllReduce
    python -m nano_nccl_b200.bench.profile_cases gemm_rs_single | ag_gemm_single   # fused GEMM kernels, one rank, 8192 x 4096 x 1792

NANO_NCCL_PIPE_MIN_BYTES=1048576 selects the software-pipelined kernels for these cases (default: the plain kernels).

Each case also prints its CUDA-event time so the capture can be compared with an unprofiled run.
"""
from __future__ import annotations

import ctypes as C
import sys

import torch

from nano_nccl_b200 import _native as N


def _time(fn, reps=3):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(reps):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) * 1e3 / reps


def gemm():
    from nano_nccl_b200.ops.gemm import gemm_bf16, gemm_last_error

    m, n, k = 16384, 4096, 1792
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = (torch.randn(n, k, device="cuda") * 0.02).bfloat16()
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    us = _time(lambda: gemm_bf16(a, b, out=out))
    assert gemm_last_error() == 0
    print(f"gemm {m}x{n}x{k}: {us:.1f} us, {2.0 * m * n * k / us / 1e6:.0f} TFLOP/s")


def emu_twoshot():
    lib = N.load_library()
    nranks, count = 8, 16 * 1024 * 1024  # 32 MiB of bf16 per rank
    h = C.c_void_p()
    N.check(lib.nano_nccl_emu_create(0, nranks, 5_000_000, C.byref(h)))
    xs = [torch.randn(count, device="cuda").bfloat16() for _ in range(nranks)]
    outs = [torch.empty_like(x) for x in xs]
    src = (C.c_void_p * nranks)(*[x.data_ptr() for x in xs])
    dst = (C.c_void_p * nranks)(*[o.data_ptr() for o in outs])
    stream = torch.cuda.current_stream().cuda_stream

    def run():
        N.check(lib.nano_nccl_emu_all_reduce(h, src, dst, count, 2, N.REDOPS["sum"], N.ALGOS["twoshot"], 16, stream))

    us = _time(run)
    print(f"emulated two-shot all_reduce, {nranks} ranks x {count * 2 >> 20} MiB: {us:.1f} us")
    lib.nano_nccl_emu_destroy(h)


def _emu(kind: str):
    """8 emulated ranks on one GPU: the same device code as the multi-GPU kernels with every "peer"
    pointer local, so a capture shows the kernel's instruction mix and HBM traffic (not NVLink)."""
    lib = N.load_library()
    nranks, count = 8, 2 * 1024 * 1024  # per-rank chunk: 4 MiB of bf16
    h = C.c_void_p()
    N.check(lib.nano_nccl_emu_create(0, nranks, 5_000_000, C.byref(h)))
    big, small = count * nranks, count
    n_in = big if kind in ("oneshot", "reduce_scatter") else small
    n_out = big if kind in ("oneshot", "all_gather") else small
    xs = [torch.randn(n_in, device="cuda").bfloat16() for _ in range(nranks)]
    outs = [torch.empty(n_out, device="cuda", dtype=torch.bfloat16) for _ in range(nranks)]
    src = (C.c_void_p * nranks)(*[x.data_ptr() for x in xs])
    dst = (C.c_void_p * nranks)(*[o.data_ptr() for o in outs])
    stream = torch.cuda.current_stream().cuda_stream

    def run():
        if kind == "oneshot":
            N.check(lib.nano_nccl_emu_all_reduce(h, src, dst, big, 2, N.REDOPS["sum"], N.ALGOS["oneshot"], 16, stream))
        elif kind == "reduce_scatter":
            N.check(lib.nano_nccl_emu_reduce_scatter(h, src, dst, count, 2, N.REDOPS["sum"], 16, stream))
        else:
            N.check(lib.nano_nccl_emu_all_gather(h, src, dst, count, 2, 16, stream))

    us = _time(run)
    print(f"emulated {kind}, {nranks} ranks, {big * 2 >> 20} MiB buffers: {us:.1f} us")
    lib.nano_nccl_emu_destroy(h)


def emu_ll():
    """Flag-in-data one-shot AllReduce of 256 KiB on 8 emulated ranks (the small-message kernel)."""
    import os

    os.environ["NANO_NCCL_LL_MAX_BYTES"] = str(1 << 20)
    lib = N.load_library()
    nranks, count = 8, 128 * 1024  # 256 KiB of bf16 per rank
    h = C.c_void_p()
    N.check(lib.nano_nccl_emu_create(0, nranks, 5_000_000, C.byref(h)))
    xs = [torch.randn(count, device="cuda").bfloat16() for _ in range(nranks)]
    outs = [torch.empty_like(x) for x in xs]
    src = (C.c_void_p * nranks)(*[x.data_ptr() for x in xs])
    dst = (C.c_void_p * nranks)(*[o.data_ptr() for o in outs])
    stream = torch.cuda.current_stream().cuda_stream
    us = _time(lambda: N.check(lib.nano_nccl_emu_all_reduce(h, src, dst, count, 2, N.REDOPS["sum"], N.ALGOS["oneshot"], 16, stream)), reps=5)
    print(f"emulated flag-in-data all_reduce, {nranks} ranks x {count * 2 >> 10} KiB: {us:.1f} us")
    lib.nano_nccl_emu_destroy(h)


def _fused_single(which: str):
    """The fused GEMM kernels with one rank: every tile is an own tile, nothing crosses NVLink, so a capture shows
    the tensor pipe and the epilogue of the fused modes without peers."""
    from nano_nccl_b200 import Communicator
    from nano_nccl_b200.ops.gemm import FusedTensorParallel, gemm_last_error

    comm = Communicator.from_tcp("127.0.0.1", 29631, 0, 1, device=0)
    m, n, k = (8192, 4096, 1792) if which == "gemm_rs" else (8192, 1792, 4096)
    fused = FusedTensorParallel(comm, m * n * 2, m * k * 2)
    a = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(n, k, device="cuda") * 0.02).bfloat16()
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    fn = (lambda: fused.gemm_rs(a, w, out=out)) if which == "gemm_rs" else (lambda: fused.ag_gemm(a, w, out=out))
    us = _time(fn)
    assert gemm_last_error() == 0
    print(f"{which} single rank {m}x{n}x{k}: {us:.1f} us, {2.0 * m * n * k / us / 1e6:.0f} TFLOP/s")
    fused.destroy()
    comm.destroy()


def adamw():
    from nano_nccl_b200.ops.optim import adamw_step_

    n = 64 * 1024 * 1024
    p = torch.randn(n, device="cuda").bfloat16()
    g = torch.randn(n, device="cuda").bfloat16()
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    us = _time(lambda: adamw_step_(p, g, m, v, lr=1e-3, step=1))
    print(f"adamw {n} params: {us:.1f} us, {22.0 * n / us / 1e3:.0f} GB/s")


if __name__ == "__main__":
    {"gemm": gemm, "emu_twoshot": emu_twoshot, "adamw": adamw, "emu_oneshot": lambda: _emu("oneshot"),
     "emu_reduce_scatter": lambda: _emu("reduce_scatter"), "emu_all_gather": lambda: _emu("all_gather"), "emu_ll": emu_ll,
     "gemm_rs_single": lambda: _fused_single("gemm_rs"), "ag_gemm_single": lambda: _fused_single("ag_gemm")}[sys.argv[1]]()
