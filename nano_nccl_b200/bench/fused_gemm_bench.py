"""Fused tensor-parallel GEMM+collective benchmark (BF16) against cuBLAS + NCCL.

Row-parallel:    activations 8192 x (14336/N) per rank times weight (14336/N) x 4096, ReduceScatter over tokens.
Column-parallel: AllGather of (8192/N) x 4096 token shards, GEMM with a 4096 x (14336/N) weight.
Weights normal(0, 0.02), activations normal(0, 1), seeded.  5 warm-up + 20 timed iterations, CUDA events
after an L2 flush and a device-side rank alignment, p50, max over ranks.  Roofline: the slower of
FLOPs / measured bf16 GEMM peak (1667.7 TFLOP/s) and NVLink bytes / 900 GB/s (nominal, per direction);
`frac_of_roofline_measured_link` uses the bandwidth a push actually reaches on this pool instead.

Usage: torchrun --nproc-per-node N -m nano_nccl_b200.bench.fused_gemm_bench [--out file.jsonl]
       python -m nano_nccl_b200.bench.fused_gemm_bench --plain     (1 GPU: tcgen05 GEMM vs cuBLAS)

`--variants "default;NANO_NCCL_AG_PUSH_PARTS=8;NANO_NCCL_GEMM_RS_TMA=1"` times the fused kernels once per environment
variant in the same process (the switches are read when the fused workspace is created); cuBLAS + NCCL is timed once.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from nano_nccl_b200.ops.gemm import FusedTensorParallel, gemm_bf16, gemm_last_error
from nano_nccl_b200.utils.timing import L2Flusher, max_over_ranks, p50, time_iterations

PEAK_TFLOPS = 1667.7      # measured cuBLAS bf16 burst on this pool
NVLINK_GBS = 900.0        # nominal NVLink 5 bandwidth per direction per GPU: the roofline constant
NVLINK_MEASURED_GBS = 585.0  # what SM stores, TMA bulk copies and the copy engine all reach at 32 MiB (p2p_bandwidth)


def plain(args) -> None:
    torch.cuda.set_device(0)
    flush = L2Flusher()
    rows = []
    for (m, n, k) in [(8192, 4096, 1792), (8192, 1792, 4096), (8192, 8192, 8192), (8192, 4096, 14336), (4096, 4096, 4096)]:
        a = torch.randn(m, k, device="cuda").bfloat16()
        b = (torch.randn(n, k, device="cuda") * 0.02).bfloat16()
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        t_nano = p50(time_iterations(lambda: gemm_bf16(a, b, out=out), args.iters, args.warmup, flush=flush))
        t_cublas = p50(time_iterations(lambda: torch.matmul(a, b.t(), out=out), args.iters, args.warmup, flush=flush))
        assert gemm_last_error() == 0
        fl = 2.0 * m * n * k
        row = {"shape": [m, n, k], "nano_us": round(t_nano, 2), "cublas_us": round(t_cublas, 2),
               "nano_tflops": round(fl / t_nano / 1e6, 1), "cublas_tflops": round(fl / t_cublas / 1e6, 1),
               "nano_frac_of_measured_peak": round(fl / t_nano / 1e6 / PEAK_TFLOPS, 3)}
        rows.append(row)
        print(json.dumps(row), flush=True)
    if args.out:
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--plain", action="store_true")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--variants", default="", help="';'-separated environment variants of the fused kernels")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    if args.plain:
        plain(args)
        return
    from nano_nccl_b200.communicator import Communicator

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = Communicator.from_torch_distributed(device=local)
    M, H, F = args.tokens, args.hidden, args.ffn
    Fp = F // world
    from nano_nccl_b200.bench.collective_sweep import apply_variant, restore_env

    variants = [v.strip() for v in args.variants.split(";") if v.strip()] or ["default"]
    flush = L2Flusher()
    align = torch.zeros(1, device="cuda")
    torch.manual_seed(1234 + rank)

    def aligned():
        dist.all_reduce(align)

    rows = []
    # ---- row-parallel: [M, Fp] x [H, Fp]^T -> reduce-scatter over tokens -> [M/world, H]
    a = torch.randn(M, Fp, device="cuda").bfloat16()
    w = (torch.randn(H, Fp, device="cuda") * 0.02).bfloat16()
    out = torch.empty(M // world, H, device="cuda", dtype=torch.bfloat16)
    partial = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    ref_out = torch.empty_like(out)

    def baseline_rs():
        torch.matmul(a, w.t(), out=partial)
        dist.reduce_scatter_tensor(ref_out, partial)

    def fused_times(call):
        """p50 of the fused op per variant: a workspace of its own per variant, destroyed afterwards."""
        out_us = {}
        for variant in variants:
            saved = apply_variant(variant)
            tp = FusedTensorParallel(comm, M * H * 2, M * H * 2)
            restore_env(saved)
            out_us[variant] = max_over_ranks(p50(time_iterations(lambda: call(tp), args.iters, args.warmup, flush=flush, pre=aligned)))
            torch.cuda.synchronize()
            assert gemm_last_error() == 0, (variant, gemm_last_error())
            tp.destroy()
        return out_us

    rs_us = fused_times(lambda tp: tp.gemm_rs(a, w, out))
    t_fused = rs_us[variants[0]]
    t_base = max_over_ranks(p50(time_iterations(baseline_rs, args.iters, args.warmup, flush=flush, pre=aligned)))
    t_gemm = max_over_ranks(p50(time_iterations(lambda: torch.matmul(a, w.t(), out=partial), args.iters, args.warmup, flush=flush)))
    assert gemm_last_error() == 0
    err = (out.float() - ref_out.float()).abs().max().item()
    fl = 2.0 * M * H * Fp
    link_bytes = (world - 1) / world * M * H * 2
    roof_us = max(fl / (PEAK_TFLOPS * 1e6), link_bytes / (NVLINK_GBS * 1e3))
    roof_meas = max(fl / (PEAK_TFLOPS * 1e6), link_bytes / (NVLINK_MEASURED_GBS * 1e3))
    rows.append({"op": "gemm_rs", "nranks": world, "M": M, "N": H, "K_per_rank": Fp, "fused_us": round(t_fused, 2),
                 "cublas_nccl_us": round(t_base, 2), "cublas_only_us": round(t_gemm, 2), "roofline_us": round(roof_us, 2),
                 "frac_of_roofline": round(roof_us / t_fused, 3), "frac_of_roofline_measured_link": round(roof_meas / t_fused, 3),
                 "speedup_vs_cublas_nccl": round(t_base / t_fused, 3), "max_abs_diff_vs_baseline": round(err, 4),
                 "variants_us": {k: round(v, 2) for k, v in rs_us.items()}})
    # ---- column-parallel: all-gather [M/world, H] shards -> [M, H] x [Fp, H]^T -> [M, Fp]
    x = torch.randn(M // world, H, device="cuda").bfloat16()
    w2 = (torch.randn(Fp, H, device="cuda") * 0.02).bfloat16()
    out2 = torch.empty(M, Fp, device="cuda", dtype=torch.bfloat16)
    gathered = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    ref2 = torch.empty_like(out2)

    def baseline_ag():
        dist.all_gather_into_tensor(gathered, x)
        torch.matmul(gathered, w2.t(), out=ref2)

    ag_us = fused_times(lambda tp: tp.ag_gemm(x, w2, out2))
    t_fused2 = ag_us[variants[0]]
    t_base2 = max_over_ranks(p50(time_iterations(baseline_ag, args.iters, args.warmup, flush=flush, pre=aligned)))
    assert gemm_last_error() == 0
    err2 = (out2.float() - ref2.float()).abs().max().item()
    fl2 = 2.0 * M * H * Fp
    link2 = (world - 1) / world * M * H * 2
    roof2 = max(fl2 / (PEAK_TFLOPS * 1e6), link2 / (NVLINK_GBS * 1e3))
    roof2_meas = max(fl2 / (PEAK_TFLOPS * 1e6), link2 / (NVLINK_MEASURED_GBS * 1e3))
    rows.append({"op": "ag_gemm", "nranks": world, "M": M, "N_per_rank": Fp, "K": H, "fused_us": round(t_fused2, 2),
                 "cublas_nccl_us": round(t_base2, 2), "roofline_us": round(roof2, 2),
                 "frac_of_roofline": round(roof2 / t_fused2, 3), "frac_of_roofline_measured_link": round(roof2_meas / t_fused2, 3),
                 "speedup_vs_cublas_nccl": round(t_base2 / t_fused2, 3), "max_abs_diff_vs_baseline": round(err2, 4),
                 "variants_us": {k: round(v, 2) for k, v in ag_us.items()}})
    if rank == 0:
        for r in rows:
            print(json.dumps(r), flush=True)
        if args.out:
            os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
            with open(args.out, "w") as f:
                for r in rows:
                    f.write(json.dumps(r) + "\n")
    comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
