"""Multi-GPU collectives, one process per GPU (skipped below 2 GPUs)."""
import pytest

from _spawn import run_ranks
from conftest import gpu_count

pytestmark = pytest.mark.gpu


def _ranks():
    n = gpu_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    return 8 if n >= 8 else 4 if n >= 4 else 2


@pytest.mark.parametrize("mode", ["matrix", "nan", "invalid", "symmetric", "large", "symmetric_rs_ag", "symmetric_pool",
                                  "registered", "graph"])
def test_collective_matrix(mode):
    outs = run_ranks("collective_worker.py", _ranks(), [mode], timeout=600)
    assert all(f"{mode} ok" in o for o in outs), outs
