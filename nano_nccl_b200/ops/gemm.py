"""tcgen05 BF16 GEMM and the fused tensor-parallel GEMM+collective ops (tensor-level wrappers)."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _native as N


def _check_bf16(*ts):
    for t in ts:
        if t is not None and not (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()):
            raise ValueError("expected contiguous bfloat16 CUDA tensors")


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None,
              out: Optional[torch.Tensor] = None, max_ctas: int = 0) -> torch.Tensor:
    """out[M,N] = a[M,K] @ b[N,K].T (+ bias): hand-written tcgen05 / TMEM / TMA kernel."""
    _check_bf16(a, b, bias)
    m, k = a.shape
    n, k2 = b.shape
    if k != k2:
        raise ValueError("inner dimensions differ")
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    lib = N.load_library()
    N.check(lib.nano_nccl_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(),
                                    bias.data_ptr() if bias is not None else None, m, n, k,
                                    torch.cuda.current_stream().cuda_stream, max_ctas))
    return out


def gemm_last_error(device: Optional[int] = None) -> int:
    lib = N.load_library()
    return lib.nano_nccl_gemm_last_error(torch.cuda.current_device() if device is None else device)


class FusedTensorParallel:
    """Workspace + entry points of GEMM->ReduceScatter and AllGather->GEMM on one communicator."""

    def __init__(self, comm, max_rs_bytes: int, max_ag_bytes: int):
        self._lib = N.load_library()
        self.comm = comm
        h = C.c_void_p()
        N.check(self._lib.nano_nccl_fused_gemm_create(C.c_void_p(comm.handle), max_rs_bytes, max_ag_bytes, C.byref(h)))
        self._h = h

    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """a[M,Kp] (this rank's K slice) @ w[N,Kp].T, summed over ranks, rows scattered: out[M/R, N]."""
        _check_bf16(a, w)
        m, kp = a.shape
        n = w.shape[0]
        if out is None:
            out = torch.empty((m // self.comm.size, n), dtype=torch.bfloat16, device=a.device)
        N.check(self._lib.nano_nccl_gemm_rs(self._h, a.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, kp,
                                            torch.cuda.current_stream().cuda_stream))
        return out

    def ag_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                push_ctas: int = 0) -> torch.Tensor:
        """AllGather(x_shard[M/R,K]) @ w[Np,K].T -> out[M, Np]."""
        _check_bf16(x_shard, w)
        rows, k = x_shard.shape
        m = rows * self.comm.size
        np_ = w.shape[0]
        if out is None:
            out = torch.empty((m, np_), dtype=torch.bfloat16, device=x_shard.device)
        N.check(self._lib.nano_nccl_ag_gemm(self._h, x_shard.data_ptr(), w.data_ptr(), out.data_ptr(), m, np_, k,
                                            torch.cuda.current_stream().cuda_stream, push_ctas))
        return out

    def read_trace(self):
        """Time line of the last fused call as {cta: {"epilogue": [(tag, ns), ...], "producer": [...]}}; needs
        NANO_NCCL_GEMM_TRACE=1 in the environment when this object was created (empty dict otherwise).
        Tags: 0 kernel entry, 1 accumulator complete, 2 peers' partials arrived, 3 accumulator handed back,
        5 / 6 producer starts / ends waiting for a remote row block (AllGather->GEMM); in GEMM->ReduceScatter the
        "producer" list is the flag publisher's: 7 a foreign tile's stores all issued, 4 its flag published."""
        cap = (256 + 64) * 2 * 128
        buf = (C.c_ulonglong * cap)()
        n = C.c_size_t(0)
        N.check(self._lib.nano_nccl_fused_gemm_read_trace(self._h, buf, cap, C.byref(n)))
        out = {}
        mask = (1 << 60) - 1
        for cta in range(n.value // 256):
            roles = {}
            for role, name in ((0, "epilogue"), (1, "producer")):
                words = [buf[(cta * 2 + role) * 128 + i] for i in range(128)]
                events = [(w >> 60, w & mask) for w in words if w != 0]
                if events:
                    roles[name] = events
            if roles:
                out[cta] = roles
        return out

    def destroy(self):
        if self._h is not None:
            h, self._h = self._h, None
            N.check(self._lib.nano_nccl_fused_gemm_destroy(h))
