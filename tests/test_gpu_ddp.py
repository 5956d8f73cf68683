"""Data-parallel engine on 2+ GPUs."""
import pytest

from _spawn import run_ranks
from conftest import multi_gpu_ranks

pytestmark = pytest.mark.gpu


def test_data_parallel_gradients_match_reference():
    outs = run_ranks("ddp_worker.py", multi_gpu_ranks(4), timeout=300)
    assert all("ddp ok" in o for o in outs), outs


def test_optimizer_state_sharding_matches_the_replicated_engine():
    outs = run_ranks("ddp_shard_worker.py", multi_gpu_ranks(4), timeout=300)
    assert all("ok" in o for o in outs), outs
