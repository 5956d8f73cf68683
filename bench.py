#!/usr/bin/env python
"""Headline benchmark: the data-parallel GPT-2-medium training step (BF16, seq 1024, micro-batch
8 per GPU, 25 MB gradient buckets AllReduced with avg through this framework's kernels, overlapped
with backward), reported as whole-job tokens/s.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Rank 0 prints one JSON line.  `value` is timed on the device (CUDA events, max over ranks) with
the inputs already resident; `e2e` times the same K steps through the public API including the
pinned-host -> device copy of every step's tokens and the device -> host read of every step's
loss.

At 2 or more GPUs the line also carries `collectives`: the AllReduce / ReduceScatter / AllGather grid
(float, fp16, bf16; 256 KiB .. 64 MiB x4; sum) measured in the same process right after the training
steps, for this library and for NCCL, timed on the device (p50, max over ranks), plus `native_table`,
this library's native benchmark programs run with the reference's host-timed loop.  `--impl reference`
runs the unmodified reference's own benchmark programs (baseline/reference_arm.py) on the same grid at
every channel count it is built for and reports them under the same key; the reference has no model and
no one-rank mode, so its tokens/s value stays `unavailable`.  `--mode collectives` skips the training
steps and makes the grid's geomean bus bandwidth the headline value.  `--impl ddp_nccl` is torch
DistributedDataParallel over NCCL, `--impl ddp_nano` the same over this library's c10d backend "nano".
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="nano", choices=["nano", "reference", "ddp_nccl", "ddp_nano"])
    ap.add_argument("--mode", default="train", choices=["train", "collectives"],
                    help="collectives: no training steps, the headline value is the grid's geomean bus bandwidth")
    ap.add_argument("--no-collectives", action="store_true", help="train mode: skip the collective grid after the steps")
    ap.add_argument("--no-native-table", action="store_true", help="skip the host-timed run of the native benchmark programs")
    ap.add_argument("--ref-budget-s", type=float, default=240.0, help="time budget of the reference's benchmark programs")
    ap.add_argument("--model", default="gpt2-medium")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--no-overlap", action="store_true")
    ap.add_argument("--comm-ctas", type=int, default=-1, help="CTAs of a gradient reduction beside backward (-1: the engine's default, 0: the tuner's grid)")
    ap.add_argument("--shard-optimizer", action="store_true",
                    help="optimizer-state sharding: ReduceScatter + AdamW on 1/N + AllGather instead of AllReduce + AdamW")
    ap.add_argument("--extras-deadline-s", type=float, default=420.0,
                    help="every rank exits (0) this long after the timed steps if the extra measurements are stuck")
    ap.add_argument("--no-tail-full-grid", action="store_true",
                    help="keep the few-CTA grid also for the last gradient bucket (nothing overlaps with it)")
    ap.add_argument("--nano-linear", action="store_true", help="forward GEMMs of the linear layers on the tcgen05 kernel")
    return ap.parse_args()


METRIC_TRAIN = "DP training tokens/s, GPT-2-medium, BF16 (collectives: AllReduce avg of 25 MB buckets)"
METRIC_COLLECTIVES = "AllReduce/RS/AG bus GB/s (geomean over float/fp16/bf16 x 256 KiB..64 MiB x4, sum) + p50 us per cell"
PUBLISHED_GEOMEAN_VS_NCCL = 1.10  # the reference's published geomean of NCCL time / its own time (other hardware)


def reference_arm(args) -> None:
    """The unmodified reference: its own benchmark programs on the collective grid (2, 4 or 8 GPUs); no
    tokens/s value, because it has no model, no torch binding and no one-rank mode.  Under torchrun only
    rank 0 works: the programs start their own ranks, one per GPU, under the bundled launcher."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from baseline.reference_arm import run_reference

    out = run_reference(args.gpus, args.steps, args.warmup, budget_s=args.ref_budget_s)
    if args.mode == "collectives":
        coll = out.get("collectives", {})
        out.update({"metric": METRIC_COLLECTIVES, "value": coll.get("best_geomean_busbw_gbs"), "unit": "GB/s",
                    "higher_is_better": True, "dtype": "float/fp16/bf16"})
        if out["value"] is not None:
            out.pop("unavailable", None)
    print(json.dumps(out), flush=True)


def collectives_only(args, rank, world, local, dev) -> None:
    """--mode collectives: the grid is the whole benchmark; value = geomean bus bandwidth of this library."""
    import torch
    import torch.distributed as dist

    from nano_nccl_b200 import _native
    from nano_nccl_b200.bench.headline import collective_grid, native_table
    from nano_nccl_b200.communicator import Communicator
    from nano_nccl_b200.utils.timing import ClockSampler

    if world < 2:
        raise SystemExit("--mode collectives needs 2 or more GPUs (a collective between one rank is a copy)")
    comm = Communicator.from_torch_distributed(device=local)
    sampler = ClockSampler(gpu_index=local).start() if rank == 0 else None
    grid = collective_grid(comm, world, iters=max(20, args.steps), warmup=max(5, args.warmup))
    clocks = sampler.stop() if sampler is not None else None
    comm.destroy()
    dist.destroy_process_group()
    if rank != 0:
        return
    ratio = grid.get("geomean_nccl_time_over_nano_time")
    out = {"metric": METRIC_COLLECTIVES, "value": grid["geomean_busbw_gbs"], "unit": "GB/s", "n_gpus": world,
           "steps": max(20, args.steps), "warmup": max(5, args.warmup), "ms_per_step": None, "higher_is_better": True,
           "scaling": "weak", "vs_baseline": round(ratio / PUBLISHED_GEOMEAN_VS_NCCL, 4) if ratio else None,
           "dtype": "float/fp16/bf16", "data": "synthetic, uniform[-1,1) seeded per rank", "impl": "nano",
           "config": {"grid": "AR/RS/AG x float,fp16,bf16 x 256KiB..64MiB x4, sum", "l2": "flushed between iterations",
                      "parallelism": f"{world} ranks, one per GPU"},
           "gpu_launches": grid["nano_kernel_launches"], "clocks": clocks, "collectives": grid,
           "native_library": _native.library_loaded_path()}
    if not args.no_native_table:
        out["collectives"]["native_table"] = native_table(world)
    print(json.dumps(out), flush=True)


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from nano_nccl_b200.models.gpt2 import PRESETS, build
    from nano_nccl_b200.utils.timing import ClockSampler

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)  # control plane: barriers and the max over ranks of the timings
    if args.mode == "collectives":
        collectives_only(args, rank, world, local, dev)
        return
    cfg = PRESETS[args.model]
    model = build(args.model, device=dev, dtype=torch.bfloat16, seed=0)
    mb, seq = args.micro_batch, cfg.seq_len
    tokens_per_step = mb * seq * world
    nano_linears = 0
    if args.nano_linear and args.impl == "nano":
        from nano_nccl_b200.ops.linear import use_nano_linear

        nano_linears = use_nano_linear(model)

    if args.impl == "nano":
        from nano_nccl_b200.communicator import Communicator
        from nano_nccl_b200.parallel.ddp import DataParallel

        if world > 1:
            comm = Communicator.from_torch_distributed(device=local)
        engine = DataParallel(model, comm, bucket_bytes=25 * 1024 * 1024, overlap=not args.no_overlap,
                              comm_ctas=None if args.comm_ctas < 0 else args.comm_ctas, tail_full_grid=not args.no_tail_full_grid,
                              shard_optimizer=args.shard_optimizer)

        def train_step(idx, tgt):
            engine.zero_grad()
            loss = engine(idx, tgt)
            loss.backward()
            engine.step()
            return loss

        launches_per_step = engine.launches_per_step() + nano_linears
    else:  # torch DDP (over NCCL, or over this library's c10d backend) with torch's fused AdamW
        group = None
        if world > 1 and args.impl == "ddp_nano":
            import nano_nccl_b200.parallel.process_group  # noqa: F401  (registers the c10d backend "nano")

            group = dist.new_group(backend="nano")  # gradients, buffers and the initial broadcast go through this library
        ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], bucket_cap_mb=25, process_group=group,
                                                        gradient_as_bucket_view=True) if world > 1 else model
        opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)

        def train_step(idx, tgt):
            opt.zero_grad(set_to_none=True)
            loss = ddp(idx, tgt)
            loss.backward()
            opt.step()
            return loss

        launches_per_step = 0

    # synthetic data: token ids uniform over the vocabulary, a pool of pinned host batches
    g = torch.Generator().manual_seed(1234 + rank)
    pool = 4
    host_idx = [torch.randint(0, cfg.vocab_size, (mb, seq), generator=g).pin_memory() for _ in range(pool)]
    host_tgt = [torch.randint(0, cfg.vocab_size, (mb, seq), generator=g).pin_memory() for _ in range(pool)]
    dev_idx = [t.to(dev) for t in host_idx]
    dev_tgt = [t.to(dev) for t in host_tgt]
    host_loss = torch.zeros(1, dtype=torch.float32).pin_memory()

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (shared by both measurements)
    for i in range(max(3, args.warmup)):
        train_step(dev_idx[i % pool], dev_tgt[i % pool])
    sync_all()

    # ---- measurement 1: device-timed, inputs resident
    sampler = ClockSampler(gpu_index=local).start() if rank == 0 else None
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    start.record()
    for i in range(args.steps):
        loss = train_step(dev_idx[i % pool], dev_tgt[i % pool])
    stop.record()
    sync_all()
    dev_ms = start.elapsed_time(stop)
    final_loss = float(loss.detach())

    # ---- measurement 2: end to end (H2D of every step's tokens, D2H of every step's loss)
    idx_buf = torch.empty((mb, seq), dtype=torch.long, device=dev)
    tgt_buf = torch.empty((mb, seq), dtype=torch.long, device=dev)
    sync_all()
    t0 = time.perf_counter()
    for i in range(args.steps):
        idx_buf.copy_(host_idx[i % pool], non_blocking=True)
        tgt_buf.copy_(host_tgt[i % pool], non_blocking=True)
        loss = train_step(idx_buf, tgt_buf)
        host_loss.copy_(loss.detach().float().reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the loss value is on the host now
    sync_all()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop() if sampler is not None else None

    def reduce_max(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    dev_ms = reduce_max(dev_ms)
    e2e_ms = reduce_max(e2e_ms)
    out = None
    if rank == 0:
        from nano_nccl_b200 import _native

        value = tokens_per_step * args.steps / (dev_ms / 1e3)
        e2e_value = tokens_per_step * args.steps / (e2e_ms / 1e3)
        out = {
            "metric": METRIC_TRAIN,
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": round(dev_ms / args.steps, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic token ids (uniform over vocab), random-init weights", "impl": args.impl,
            "config": {"model": args.model, "global_batch": mb * world, "seq_len": seq,
                       "parallelism": f"dp{world}", "bucket_mb": 25, "optimizer": "fused AdamW",
                       "l2": "step working set (weights + activations, several GB) far exceeds the 126 MB L2",
                       "overlap": not args.no_overlap},
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms / args.steps, 3),
                    "h2d_bytes_per_step": 2 * mb * seq * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks, "final_loss": round(final_loss, 4),
            "native_library": _native.library_loaded_path(),
        }

    # Everything below adds detail to the line and is not part of the timed measurement.  It must never cost the
    # line itself: an error is recorded in the line, and a deadline ends every rank (exit 0, rank 0 prints what it
    # has) if a rank is stuck in a collective that its peers have left.
    import threading

    printed = threading.Event()

    def emit(note: str | None = None) -> None:
        if rank == 0 and not printed.is_set():
            printed.set()
            if note is not None:
                out.setdefault("notes", []).append(note)
            print(json.dumps(out), flush=True)

    def deadline_passed() -> None:
        emit(f"the measurements after the timed steps did not finish within {args.extras_deadline_s} s")
        os._exit(0)

    watchdog = threading.Timer(args.extras_deadline_s, deadline_passed)
    watchdog.daemon = True
    watchdog.start()
    collectives = None
    try:
        if args.impl == "nano":   # three more steps with events around every bucket's reduction (not timed above)
            engine.enable_timeline(True)
            for i in range(3):
                train_step(dev_idx[i % pool], dev_tgt[i % pool])
            breakdown = engine.timeline_summary()
            engine.enable_timeline(False)
            if out is not None:
                out["step_breakdown"] = breakdown
        if world > 1 and args.impl == "nano" and not args.no_collectives:
            from nano_nccl_b200.bench.headline import collective_grid

            comm.set_grid_override(0)
            collectives = collective_grid(comm, world)
            if out is not None:
                out["collectives"] = collectives
                out["gpu_launches_collective_grid"] = collectives["nano_kernel_launches"]
        if comm is not None:
            comm.destroy()
            comm = None
        if world > 1:
            dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001 - the line is printed with the error in it; peers leave at the deadline
        emit(f"after the timed steps: {type(e).__name__}: {str(e)[:300]}")
        os._exit(0)
    watchdog.cancel()
    if rank == 0:
        if collectives is not None and not args.no_native_table:
            from nano_nccl_b200.bench.headline import native_table

            try:
                collectives["native_table"] = native_table(world)
            except Exception as e:  # noqa: BLE001
                collectives["native_table"] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
        emit()


if __name__ == "__main__":
    main()
