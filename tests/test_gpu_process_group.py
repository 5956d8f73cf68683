"""The c10d backend "nano" (C++ extension) on 2+ GPUs."""
import pytest

from _spawn import run_ranks
from conftest import multi_gpu_ranks

pytestmark = pytest.mark.gpu


def test_c10d_backend_and_torch_ops():
    outs = run_ranks("pg_worker.py", multi_gpu_ranks(4), timeout=300)
    assert all("pg ok" in o for o in outs), outs


def test_torch_ops_gemm_and_fused_collectives():
    outs = run_ranks("torch_ops_worker.py", multi_gpu_ranks(4), timeout=300)
    assert all("ok" in o for o in outs), outs
