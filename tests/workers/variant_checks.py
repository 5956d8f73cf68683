"""Single-GPU checks of kernel variants that are selected by an environment variable or a run-time argument
(each case is one process, so the variable is set before the library reads it):

    bulk_copy          TMA bulk-copy, vector-copy and copy-engine push kernels, local destinations
    emu_tma_allgather  AllGather whose pushes are TMA bulk copies (NANO_NCCL_PUSH_TMA=1), 2 / 4 / 8 emulated ranks
    emu_ll             flag-in-data small-message kernels (NANO_NCCL_LL_MAX_BYTES), 2 / 4 / 8 emulated ranks
    fused_single       plain GEMM and the fused GEMM kernels with one rank and every tile width
    emu_pipe           software-pipelined large-message kernels (AllReduce two-shot, ReduceScatter, AllGather) with
                       small tiles so that a CTA walks many of them, interleaved with the plain kernels

Each check compares against a plain PyTorch result, uses guard bands, and relies on the kernels' bounded waits.
tests/test_gpu_variants.py runs them.
"""
import ctypes as C
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

import torch  # noqa: E402

from nano_nccl_b200 import _native as N  # noqa: E402

GUARD = 64
SENTINEL = 77


def bulk_copy():
    lib = N.load_library()
    stream = torch.cuda.current_stream().cuda_stream
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    for nbytes in (16, 4096, 16 * 1024, 16 * 1024 + 16, 1_000_000 // 16 * 16, 5 * 1024 * 1024 + 48):
        src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda")
        for engine, ctas, chunk, stages in [(1, 3, 0, 0), (2, 1, 0, 0), (0, 1, 4096, 3), (0, 2, 16384, 6), (0, 7, 8192, 4), (0, 16, 32768, 6)]:
            outs = [torch.full((nbytes + 2 * GUARD,), SENTINEL, dtype=torch.uint8, device="cuda") for _ in range(3)]
            table = (C.c_void_p * 3)(*[o.data_ptr() + GUARD for o in outs])
            N.check(lib.nano_nccl_push_copy(engine, src.data_ptr(), table, 3, nbytes, ctas, chunk, stages, err.data_ptr(), stream))
            torch.cuda.synchronize()
            assert int(err.item()) == 0, ("device wait ran out", engine, ctas, chunk, nbytes)
            for o in outs:
                assert torch.equal(o[GUARD:GUARD + nbytes], src), ("content", engine, ctas, chunk, nbytes)
                assert (o[:GUARD] == SENTINEL).all() and (o[-GUARD:] == SENTINEL).all(), ("guard band", engine, nbytes)
    print("bulk_copy ok")


def emu_tma_allgather():
    os.environ["NANO_NCCL_PUSH_TMA"] = "1"
    lib = N.load_library()
    stream = torch.cuda.current_stream().cuda_stream
    for nranks in (2, 4, 8):
        h = C.c_void_p()
        N.check(lib.nano_nccl_emu_create(0, nranks, 5_000_000, C.byref(h)))
        try:
            for dtype, code in ((torch.float32, 0), (torch.bfloat16, 2)):
                for count in (8, 4096, 70000, 1024 * 1024 + 8):
                    for rounds in range(2):  # both staging halves
                        xs = [torch.randn(count, device="cuda").to(dtype) for _ in range(nranks)]
                        fulls = [torch.full((count * nranks + 2 * GUARD,), float(SENTINEL), dtype=dtype, device="cuda")
                                 for _ in range(nranks)]
                        outs = [f[GUARD:GUARD + count * nranks] for f in fulls]
                        src = (C.c_void_p * nranks)(*[x.data_ptr() for x in xs])
                        dst = (C.c_void_p * nranks)(*[o.data_ptr() for o in outs])
                        N.check(lib.nano_nccl_emu_all_gather(h, src, dst, count, code, 12, stream))
                        torch.cuda.synchronize()
                        words = (C.c_uint32 * 4)()
                        for r in range(nranks):
                            N.check(lib.nano_nccl_emu_status(h, r, words))
                            assert words[0] == 0, ("device status", r, list(words))
                        want = torch.cat(xs)
                        for f, o in zip(fulls, outs):
                            assert torch.equal(o, want), ("content", nranks, dtype, count)
                            assert (f[:GUARD] == SENTINEL).all() and (f[-GUARD:] == SENTINEL).all(), "guard band"
        finally:
            lib.nano_nccl_emu_destroy(h)
    print("emu_tma_allgather ok")


def emu_ll():
    """Flag-in-data (LL) AllReduce / ReduceScatter / AllGather on emulated ranks against PyTorch."""
    os.environ["NANO_NCCL_LL_MAX_BYTES"] = str(1 << 20)
    lib = N.load_library()
    stream = torch.cuda.current_stream().cuda_stream
    tol = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}
    code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

    def ref(xs, op):
        acc = torch.stack([x.float() for x in xs])
        return {"sum": acc.sum(0), "avg": acc.sum(0) / len(xs), "max": acc.max(0).values, "min": acc.min(0).values}[op]

    def guarded(n, dtype):
        full = torch.full((n + 2 * GUARD,), float(SENTINEL), dtype=dtype, device="cuda")
        return full, full[GUARD:GUARD + n]

    def clean(h, nranks):
        words = (C.c_uint32 * 4)()
        for r in range(nranks):
            N.check(lib.nano_nccl_emu_status(h, r, words))
            assert words[0] == 0, ("device status", r, list(words))

    for nranks in (2, 4, 8):
        h = C.c_void_p()
        N.check(lib.nano_nccl_emu_create(0, nranks, 5_000_000, C.byref(h)))
        try:
            for dtype in (torch.float32, torch.float16, torch.bfloat16):
                for count in (1, 5, 17, 4099, 20000):
                    for op in ("sum", "avg", "max", "min"):
                        for _ in range(3):  # both staging halves and a reuse
                            xs = [(torch.rand(count, device="cuda") * 2 - 1).to(dtype) for _ in range(nranks)]
                            outs = [guarded(count, dtype) for _ in range(nranks)]
                            src = (C.c_void_p * nranks)(*[x.data_ptr() for x in xs])
                            dst = (C.c_void_p * nranks)(*[o[1].data_ptr() for o in outs])
                            N.check(lib.nano_nccl_emu_all_reduce(h, src, dst, count, code[dtype], N.REDOPS[op],
                                                                 N.ALGOS["oneshot"], 12, stream))
                            torch.cuda.synchronize()
                            clean(h, nranks)
                            want = ref(xs, op).to(dtype).float()
                            for full, out in outs:
                                assert ((out.float() - want).abs() <= tol[dtype] * want.abs().clamp(min=1)).all(), ("ar", nranks, dtype, count, op)
                                assert (full[:GUARD] == SENTINEL).all() and (full[-GUARD:] == SENTINEL).all()
                        xs = [(torch.rand(count * nranks, device="cuda") * 2 - 1).to(dtype) for _ in range(nranks)]
                        outs = [guarded(count, dtype) for _ in range(nranks)]
                        src = (C.c_void_p * nranks)(*[x.data_ptr() for x in xs])
                        dst = (C.c_void_p * nranks)(*[o[1].data_ptr() for o in outs])
                        N.check(lib.nano_nccl_emu_reduce_scatter(h, src, dst, count, code[dtype], N.REDOPS[op], 12, stream))
                        torch.cuda.synchronize()
                        clean(h, nranks)
                        want = ref(xs, op).to(dtype).float()
                        for r, (full, out) in enumerate(outs):
                            w = want[r * count:(r + 1) * count]
                            assert ((out.float() - w).abs() <= tol[dtype] * w.abs().clamp(min=1)).all(), ("rs", nranks, dtype, count, op)
                            assert (full[:GUARD] == SENTINEL).all() and (full[-GUARD:] == SENTINEL).all()
                    if dtype != torch.float16:
                        xs = [(torch.rand(count, device="cuda") * 2 - 1).to(dtype) for _ in range(nranks)]
                        outs = [guarded(count * nranks, dtype) for _ in range(nranks)]
                        src = (C.c_void_p * nranks)(*[x.data_ptr() for x in xs])
                        dst = (C.c_void_p * nranks)(*[o[1].data_ptr() for o in outs])
                        N.check(lib.nano_nccl_emu_all_gather(h, src, dst, count, code[dtype], 12, stream))
                        torch.cuda.synchronize()
                        clean(h, nranks)
                        want = torch.cat(xs)
                        for full, out in outs:
                            assert torch.equal(out, want), ("ag", nranks, dtype, count)
                            assert (full[:GUARD] == SENTINEL).all() and (full[-GUARD:] == SENTINEL).all()
        finally:
            lib.nano_nccl_emu_destroy(h)
    del os.environ["NANO_NCCL_LL_MAX_BYTES"]
    print("emu_ll ok")


def emu_pipe():
    """Pipelined kernels on emulated ranks: messages of 64 KiB and more take them (4 KiB tiles, so every CTA walks
    many tiles and every buffer is reused several times); smaller messages in between take the plain kernels on
    the same staging memory, which exercises the barriers at both ends of a pipelined kernel."""
    os.environ["NANO_NCCL_PIPE_MIN_BYTES"] = str(64 * 1024)
    os.environ["NANO_NCCL_PIPE_TILE_BYTES"] = "4096"
    os.environ["NANO_NCCL_PIPE_DEPTH"] = os.environ.get("NANO_TEST_PIPE_DEPTH", "0")   # 0: the built-in depth
    lib = N.load_library()
    stream = torch.cuda.current_stream().cuda_stream
    tol = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}
    code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

    def ref(xs, op):
        acc = torch.stack([x.float() for x in xs])
        return {"sum": acc.sum(0), "avg": acc.sum(0) / len(xs), "max": acc.max(0).values, "min": acc.min(0).values}[op]

    def guarded(n, dtype):
        full = torch.full((n + 2 * GUARD,), float(SENTINEL), dtype=dtype, device="cuda")
        return full, full[GUARD:GUARD + n]

    def clean(h, nranks):
        words = (C.c_uint32 * 4)()
        for r in range(nranks):
            N.check(lib.nano_nccl_emu_status(h, r, words))
            assert words[0] == 0, ("device status", r, list(words))

    quick = os.environ.get("NANO_TEST_PIPE_DEPTH", "0") != "0"   # the other depths: a smaller matrix
    for nranks in ((2, 8) if quick else (2, 3, 4, 8)):
        h = C.c_void_p()
        N.check(lib.nano_nccl_emu_create(0, nranks, 5_000_000, C.byref(h)))
        try:
            for dtype in ((torch.float32, torch.bfloat16) if quick else (torch.float32, torch.bfloat16, torch.float16)):
                esz = torch.empty((), dtype=dtype).element_size()
                # below the threshold (plain), just above, odd and unaligned, several tiles per CTA, a large one
                for count in ((1000, 70001, 300_003) if quick else (1000, 64 * 1024 // esz, 70001, 300_003, 1_500_000)):
                    for op in (("sum", "max") if count > 100000 else ("sum", "avg", "max", "min")):
                        xs = [(torch.rand(count, device="cuda") * 2 - 1).to(dtype) for _ in range(nranks)]
                        outs = [guarded(count, dtype) for _ in range(nranks)]
                        src = (C.c_void_p * nranks)(*[x.data_ptr() for x in xs])
                        dst = (C.c_void_p * nranks)(*[o[1].data_ptr() for o in outs])
                        N.check(lib.nano_nccl_emu_all_reduce(h, src, dst, count, code[dtype], N.REDOPS[op],
                                                             N.ALGOS["twoshot"], 12, stream))
                        torch.cuda.synchronize()
                        clean(h, nranks)
                        want = ref(xs, op).to(dtype).float()
                        for full, out in outs:
                            assert ((out.float() - want).abs() <= tol[dtype] * want.abs().clamp(min=1)).all(), ("ar", nranks, dtype, count, op)
                            assert (full[:GUARD] == SENTINEL).all() and (full[-GUARD:] == SENTINEL).all()
                        assert all(torch.equal(outs[0][1], o[1]) for o in outs), "ranks disagree bit-wise"
                    per = max(1, count // nranks)
                    for op in ("sum", "min"):
                        xs = [(torch.rand(per * nranks, device="cuda") * 2 - 1).to(dtype) for _ in range(nranks)]
                        outs = [guarded(per, dtype) for _ in range(nranks)]
                        src = (C.c_void_p * nranks)(*[x.data_ptr() for x in xs])
                        dst = (C.c_void_p * nranks)(*[o[1].data_ptr() for o in outs])
                        N.check(lib.nano_nccl_emu_reduce_scatter(h, src, dst, per, code[dtype], N.REDOPS[op], 12, stream))
                        torch.cuda.synchronize()
                        clean(h, nranks)
                        want = ref(xs, op).to(dtype).float()
                        for r, (full, out) in enumerate(outs):
                            w = want[r * per:(r + 1) * per]
                            assert ((out.float() - w).abs() <= tol[dtype] * w.abs().clamp(min=1)).all(), ("rs", nranks, dtype, per, op)
                            assert (full[:GUARD] == SENTINEL).all() and (full[-GUARD:] == SENTINEL).all()
                    if dtype != torch.float16:
                        xs = [(torch.rand(per, device="cuda") * 2 - 1).to(dtype) for _ in range(nranks)]
                        outs = [guarded(per * nranks, dtype) for _ in range(nranks)]
                        src = (C.c_void_p * nranks)(*[x.data_ptr() for x in xs])
                        dst = (C.c_void_p * nranks)(*[o[1].data_ptr() for o in outs])
                        N.check(lib.nano_nccl_emu_all_gather(h, src, dst, per, code[dtype], 12, stream))
                        torch.cuda.synchronize()
                        clean(h, nranks)
                        want = torch.cat(xs)
                        for full, out in outs:
                            assert torch.equal(out, want), ("ag", nranks, dtype, per)
                            assert (full[:GUARD] == SENTINEL).all() and (full[-GUARD:] == SENTINEL).all()
        finally:
            lib.nano_nccl_emu_destroy(h)
    del os.environ["NANO_NCCL_PIPE_MIN_BYTES"], os.environ["NANO_NCCL_PIPE_TILE_BYTES"], os.environ["NANO_NCCL_PIPE_DEPTH"]
    print("emu_pipe ok")


def fused_single():
    """The fused GEMM kernels with ONE rank (all tiles are own tiles, nothing crosses NVLink) and the plain GEMM,
    with the run-time tile widths, against fp32 products."""
    from nano_nccl_b200 import Communicator
    from nano_nccl_b200.ops.gemm import FusedTensorParallel, gemm_bf16, gemm_last_error

    comm = Communicator.from_tcp("127.0.0.1", 29611, 0, 1, device=0)
    for setting in ("", "224", "192", "auto"):
        if setting:
            os.environ["NANO_NCCL_GEMM_BN"] = setting
        else:
            os.environ.pop("NANO_NCCL_GEMM_BN", None)
        fused = FusedTensorParallel(comm, 1024 * 2048 * 2, 1024 * 2048 * 2)
        for (m, n, k) in ((256, 512, 128), (1024, 1792, 512), (384, 264, 72), (1024, 2048, 64)):
            a = torch.randn(m, k, device="cuda").bfloat16()
            w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
            want = a.float() @ w.float().t()
            tol = 2e-2 * want.abs().clamp(min=1.0)
            for name, got in (("gemm", gemm_bf16(a, w)), ("gemm_rs", fused.gemm_rs(a, w)), ("ag_gemm", fused.ag_gemm(a, w))):
                torch.cuda.synchronize()
                assert gemm_last_error() == 0, (name, setting, gemm_last_error())
                assert bool(((got.float() - want).abs() <= tol).all()), (name, setting, (m, n, k))
        fused.destroy()
    os.environ.pop("NANO_NCCL_GEMM_BN", None)
    comm.destroy()
    print("fused_single ok")


if __name__ == "__main__":
    which = sys.argv[1] if len(sys.argv) > 1 else "all"
    if which in ("bulk_copy", "all"):
        bulk_copy()
    if which in ("emu_tma_allgather", "all"):
        emu_tma_allgather()
    if which in ("emu_ll", "all"):
        emu_ll()
    if which in ("fused_single", "all"):
        fused_single()
    if which in ("emu_pipe", "all"):
        emu_pipe()
