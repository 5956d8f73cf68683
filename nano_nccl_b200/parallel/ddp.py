"""Data-parallel training engine: flat gradient buckets in symmetric memory, AllReduce(avg)
launched from autograd hooks on a side stream while backward continues, fused AdamW per bucket.

No counterpart in the reference (a collective library without a framework layer); this is the
"data-parallel gradient AllReduce from autograd hooks, overlapped with backward" layer.

Design:
* Parameters are re-pointed into flat bf16 buffers, one per bucket (25 MB by default, filled in
  reverse parameter order, i.e. the order gradients become ready).  Gradients are views into a
  flat buffer per bucket that lives in the communicator's symmetric memory, so the AllReduce is
  the zero-copy in-place NVLS kernel: no staging, the switch does the sum, the 1/N scale is fused.
* A post-accumulate-grad hook counts down the bucket; the last gradient records an event on the
  compute stream, the communication stream waits for it and launches the AllReduce.
* `step()` makes the compute stream wait for each bucket and runs one fused AdamW launch on it.
* `shard_optimizer=True` (optimizer-state sharding, "ZeRO-1"): a bucket's gradients are ReduceScattered (avg)
  instead of AllReduced, every rank keeps moments for and updates only its 1/N of the bucket, and the
  updated shards are AllGathered back into the flat parameters.  Same bytes on NVLink as the AllReduce,
  1/N of the optimizer work and of the moment memory per rank.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn as nn

from ..ops.optim import adamw_step_


@dataclass
class _Bucket:
    params: list
    numel: int
    shard_numel: int = 0              # shard_optimizer: elements of this rank's slice
    grad_shard: torch.Tensor = None   # shard_optimizer: averaged gradients of the slice
    param_shard: torch.Tensor = None  # shard_optimizer: send buffer of the parameter AllGather
    gathered: Optional[torch.cuda.Event] = None
    flat_param: torch.Tensor = None
    flat_grad: torch.Tensor = None
    m: torch.Tensor = None
    v: torch.Tensor = None
    pending: int = 0
    ready: Optional[torch.cuda.Event] = None
    done: Optional[torch.cuda.Event] = None
    launched: bool = False
    t_start: Optional[torch.cuda.Event] = None   # time line: the reduction starts on the communication stream
    t_done: Optional[torch.cuda.Event] = None    # time line: the reduction has finished


def padded_numel(numel: int) -> int:
    """Elements a bf16 parameter occupies in a flat bucket: rounded up to 8 so every parameter starts on 16 bytes."""
    return (numel + 7) // 8 * 8


def plan_buckets(numels: list, bucket_bytes: int, elem_size: int = 2) -> list:
    """Groups parameter indices into buckets in REVERSE parameter order (the order gradients become ready).
    A bucket is closed before the parameter that would push it over `bucket_bytes`; a parameter larger than
    the limit gets a bucket of its own.  Returns lists of indices into `numels`."""
    buckets, cur, cur_n = [], [], 0
    for i in reversed(range(len(numels))):
        n = padded_numel(numels[i])
        if cur and (cur_n + n) * elem_size > bucket_bytes:
            buckets.append(cur)
            cur, cur_n = [], 0
        cur.append(i)
        cur_n += n
    if cur:
        buckets.append(cur)
    return buckets


def default_comm_ctas(world: int) -> int:
    """CTAs of a gradient reduction that runs beside backward (0: the tuner's own grid).  Measured on GPT-2-medium,
    micro-batch 8 (one GPU: 32.9 ms per step).  Two B200 (peer loads, 16 in flight per thread): 8 CTAs 34.3 ms, 16: 33.8,
    32: 33.7, the tuner's 64: 33.8.  Eight B200 (in-switch reduction, where a CTA moves more): 8 CTAs 34.4 ms, 32: 34.8.
    The reduction has to be quick rather than small, because while it runs the matrix products lose those SMs and a
    whole wave with them; how many CTAs "quick" takes depends on the kernel."""
    return 32 if world <= 2 else 8


class DataParallel:
    def __init__(self, module: nn.Module, comm=None, *, bucket_bytes: int = 25 * 1024 * 1024, lr: float = 3e-4,
                 betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1, overlap: bool = True,
                 comm_ctas: Optional[int] = None, tail_full_grid: bool = True, shard_optimizer: bool = False):
        self.module = module
        self.comm = comm
        self.world = comm.size if comm is not None else 1
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.overlap = overlap
        if comm_ctas is None:
            comm_ctas = default_comm_ctas(self.world)
        self.comm_ctas = comm_ctas
        # The last bucket (the first parameters, typically the embeddings) becomes ready when backward is
        # over: nothing is left to overlap with, so its reduction may use the whole GPU.
        self.tail_full_grid = tail_full_grid
        self.shard = bool(shard_optimizer) and self.world > 1
        self.step_count = 0
        self.timeline = False
        self._t_forward = self._t_forward_end = self._t_backward_end = self._t_step_end = None
        self.collective_launches = 0
        self.optimizer_launches = 0
        params = [p for p in module.parameters() if p.requires_grad]
        if not params:
            raise ValueError("module has no trainable parameters")
        dtype = params[0].dtype
        if any(p.dtype != dtype for p in params) or dtype != torch.bfloat16:
            raise ValueError("DataParallel expects all parameters in bfloat16")
        self.device = params[0].device
        # buckets in reverse parameter order; each parameter start is 16-byte aligned
        self.buckets: list[_Bucket] = []
        for idx in plan_buckets([p.numel() for p in params], bucket_bytes):
            members = [params[i] for i in idx]
            numel = sum(padded_numel(p.numel()) for p in members)
            if shard_optimizer and self.world > 1:
                unit = 8 * self.world                     # every rank's slice starts on 16 bytes
                numel = (numel + unit - 1) // unit * unit
            self.buckets.append(_Bucket(members, numel))
        self.comm_stream = torch.cuda.Stream(priority=-1) if self.world > 1 else None
        if self.world > 1 and comm_ctas > 0:
            # The reduction runs beside backward: a few CTAs saturate NVLink, the rest of the SMs
            # stay with the GEMMs.
            comm.set_grid_override(comm_ctas)
        self._param_bucket = {}
        for b in self.buckets:
            b.flat_param = torch.empty(b.numel, dtype=dtype, device=self.device)
            if self.world > 1:
                b.flat_grad = comm.symmetric_empty(b.numel, dtype)
            else:
                b.flat_grad = torch.zeros(b.numel, dtype=dtype, device=self.device)
            if self.shard:
                b.shard_numel = b.numel // self.world
                b.grad_shard = torch.zeros(b.shard_numel, dtype=dtype, device=self.device)
                b.param_shard = torch.zeros(b.shard_numel, dtype=dtype, device=self.device)
                b.gathered = torch.cuda.Event()
            state_numel = b.shard_numel if self.shard else b.numel
            b.m = torch.zeros(state_numel, dtype=torch.float32, device=self.device)
            b.v = torch.zeros(state_numel, dtype=torch.float32, device=self.device)
            b.flat_param.zero_()
            b.ready = torch.cuda.Event()
            b.done = torch.cuda.Event()
            off = 0
            for p in b.params:
                n = p.numel()
                b.flat_param[off:off + n].view_as(p).copy_(p.data)
                p.data = b.flat_param[off:off + n].view_as(p)
                p.grad = b.flat_grad[off:off + n].view_as(p)
                self._param_bucket[p] = b
                off += padded_numel(n)
                if self.world > 1:
                    p.register_post_accumulate_grad_hook(self._hook)
        self.zero_grad()

    # ------------------------------------------------------------------ hooks
    def _hook(self, p: torch.Tensor) -> None:
        b = self._param_bucket[p]
        if b.pending <= 0 or b.launched:
            # The bucket is reduced in place: a gradient that arrives after the launch would be added on top of
            # values that are already averaged, and no second reduction would follow.
            raise RuntimeError("DataParallel: a gradient arrived for a bucket that was already reduced in this step "
                               "(a second backward without zero_grad(); gradient accumulation over several backward "
                               "passes is not supported: accumulate in the loss, or call zero_grad() between them)")
        b.pending -= 1
        if b.pending == 0 and self.overlap:
            self._launch(b)

    def _launch(self, b: _Bucket) -> None:
        b.ready.record()
        self.comm_stream.wait_event(b.ready)
        tail = self.tail_full_grid and self.comm_ctas > 0 and b is self.buckets[-1] and len(self.buckets) > 1
        if tail:
            self.comm.set_grid_override(0)   # the tuner's own grid for this size
        if self.timeline and b.t_start is not None:
            b.t_start.record(self.comm_stream)
        if self.shard:
            self.comm.reduce_scatter(b.flat_grad, b.grad_shard, "avg", stream=self.comm_stream)
        else:
            self.comm.all_reduce(b.flat_grad, b.flat_grad, "avg", stream=self.comm_stream)
        if tail:
            self.comm.set_grid_override(self.comm_ctas)
        b.done.record(self.comm_stream)
        if self.timeline:
            b.t_done.record(self.comm_stream)
        b.launched = True
        self.collective_launches += 1

    # ------------------------------------------------------------------ step API
    def zero_grad(self) -> None:
        for b in self.buckets:
            if self.comm_stream is not None and b.launched:
                torch.cuda.current_stream().wait_event(b.done)
            b.flat_grad.zero_()
            b.pending = len(b.params)
            b.launched = False

    def forward(self, *args, **kwargs):
        if not self.timeline:
            return self.module(*args, **kwargs)
        self._t_forward.record()
        out = self.module(*args, **kwargs)
        self._t_forward_end.record()
        return out

    # ------------------------------------------------------------------ time line
    def enable_timeline(self, on: bool = True) -> None:
        """Records CUDA events around every bucket's reduction and around the step, for `timeline_summary`."""
        self.timeline = bool(on)
        if self.timeline and self._t_forward is None:
            mk = lambda: torch.cuda.Event(enable_timing=True)
            self._t_forward, self._t_forward_end, self._t_backward_end, self._t_step_end = mk(), mk(), mk(), mk()
            for b in self.buckets:
                b.t_start, b.t_done = mk(), mk()

    def timeline_summary(self) -> Optional[dict]:
        """Where the last step's time went, in ms after the start of forward: when backward ended on the compute
        stream, when the optimizer finished, and for every bucket when its reduction started and ended on the
        communication stream.  `exposed_ms` is what the step spends after backward (waiting for the last
        reductions plus the optimizer); `optimizer_alone_ms` is that part without any waiting, so their difference
        is the communication that backward did not hide."""
        if not self.timeline or self.step_count == 0:
            return None
        torch.cuda.synchronize()
        t0 = self._t_forward
        bwd_end = t0.elapsed_time(self._t_backward_end)
        step_end = t0.elapsed_time(self._t_step_end)
        fwd_end = round(t0.elapsed_time(self._t_forward_end), 3)
        if self.world == 1:
            return {"forward_end_ms": fwd_end, "backward_end_ms": round(bwd_end, 3), "step_end_ms": round(step_end, 3),
                    "exposed_ms": round(step_end - bwd_end, 3)}
        rows = [{"bytes": b.numel * 2, "start_ms": round(t0.elapsed_time(b.t_start), 3),
                 "end_ms": round(t0.elapsed_time(b.t_done), 3)} for b in self.buckets]
        last_done = max(r["end_ms"] for r in rows)
        return {"forward_end_ms": fwd_end, "backward_end_ms": round(bwd_end, 3), "step_end_ms": round(step_end, 3),
                "exposed_ms": round(step_end - bwd_end, 3), "last_reduction_end_ms": round(last_done, 3),
                "reduction_after_backward_ms": round(max(0.0, last_done - bwd_end), 3),
                "reduction_busy_ms": round(sum(r["end_ms"] - r["start_ms"] for r in rows), 3), "buckets": rows}

    __call__ = forward

    def step(self) -> None:
        """Waits for each bucket's AllReduce, then runs the fused AdamW on it."""
        self.step_count += 1
        cur = torch.cuda.current_stream()
        if self.timeline:
            self._t_backward_end.record(cur)
        if self.shard and self.comm_ctas > 0:
            self.comm.set_grid_override(0)   # backward is over: the parameter gathers may use the whole GPU
        for b in self.buckets:
            if self.world > 1:
                if not b.launched:
                    self._launch(b)  # no-overlap mode, or a bucket whose hooks did not all fire
                cur.wait_event(b.done)
            if self.shard:
                lo = self.comm.rank * b.shard_numel
                mine = b.flat_param[lo:lo + b.shard_numel]
                adamw_step_(mine, b.grad_shard, b.m, b.v, lr=self.lr, betas=self.betas, eps=self.eps,
                            weight_decay=self.weight_decay, step=self.step_count, stream=cur)
                # the gather's send buffer must not overlap its receive buffer (the flat parameters)
                b.param_shard.copy_(mine)
                b.ready.record(cur)
                self.comm_stream.wait_event(b.ready)
                self.comm.all_gather(b.param_shard, b.flat_param, stream=self.comm_stream)
                b.gathered.record(self.comm_stream)
                self.collective_launches += 1
            else:
                adamw_step_(b.flat_param, b.flat_grad, b.m, b.v, lr=self.lr, betas=self.betas, eps=self.eps,
                            weight_decay=self.weight_decay, step=self.step_count, stream=cur)
            self.optimizer_launches += 1
        if self.shard:
            for b in self.buckets:   # the next forward reads the gathered parameters
                cur.wait_event(b.gathered)
            if self.comm_ctas > 0:
                self.comm.set_grid_override(self.comm_ctas)
        if self.timeline:
            self._t_step_end.record(cur)

    def launches_per_step(self) -> int:
        """Kernels of this framework launched per training step (collectives + optimizer)."""
        return len(self.buckets) * ((3 if self.shard else 2) if self.world > 1 else 1)
