"""Data-parallel engine on 2+ GPUs."""
import pytest

from _spawn import run_ranks
from conftest import gpu_count

pytestmark = pytest.mark.gpu


def test_data_parallel_gradients_match_reference():
    n = gpu_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    outs = run_ranks("ddp_worker.py", 4 if n >= 4 else 2, timeout=300)
    assert all("ddp ok" in o for o in outs), outs


def test_optimizer_state_sharding_matches_the_replicated_engine():
    n = gpu_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    outs = run_ranks("ddp_shard_worker.py", 4 if n >= 4 else 2, timeout=300)
    assert all("ok" in o for o in outs), outs
