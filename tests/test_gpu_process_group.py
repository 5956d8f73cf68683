"""The c10d backend "nano" (C++ extension) on 2+ GPUs."""
import pytest

from _spawn import run_ranks
from conftest import gpu_count

pytestmark = pytest.mark.gpu


def test_c10d_backend_and_torch_ops():
    n = gpu_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    outs = run_ranks("pg_worker.py", 4 if n >= 4 else 2, timeout=300)
    assert all("pg ok" in o for o in outs), outs


def test_torch_ops_gemm_and_fused_collectives():
    n = gpu_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    outs = run_ranks("torch_ops_worker.py", 4 if n >= 4 else 2, timeout=300)
    assert all("ok" in o for o in outs), outs
