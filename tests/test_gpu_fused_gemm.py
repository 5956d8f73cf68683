"""Fused GEMM+collective kernels on 2+ GPUs (skipped below 2 GPUs)."""
import pytest

from _spawn import run_ranks
from conftest import multi_gpu_ranks

pytestmark = pytest.mark.gpu


VARIANTS = [{}, {"NANO_NCCL_GEMM_RS_TMA": "1"}, {"NANO_NCCL_AG_GEMM_TMA": "1"}, {"NANO_NCCL_AG_PUSH_PARTS": "8"},
            {"NANO_NCCL_AG_PUSH_PARTS": "2"}, {"NANO_NCCL_GEMM_BN": "auto"}]


@pytest.mark.parametrize("env", VARIANTS, ids=lambda e: ",".join(f"{k}={v}" for k, v in e.items()) or "default")
def test_fused_gemm_collectives(env):
    ranks = multi_gpu_ranks()
    outs = run_ranks("fused_gemm_worker.py", ranks, env=env, timeout=600)
    assert all("fused ok" in o for o in outs), outs
