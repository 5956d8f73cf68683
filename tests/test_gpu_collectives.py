"""Multi-GPU collectives, one process per GPU (skipped below 2 GPUs)."""
import pytest

from _spawn import run_ranks
from conftest import multi_gpu_ranks

pytestmark = pytest.mark.gpu


def _ranks():
    return multi_gpu_ranks()


@pytest.mark.parametrize("mode", ["matrix", "nan", "invalid", "symmetric", "large", "symmetric_rs_ag", "symmetric_pool",
                                  "registered", "graph"])
def test_collective_matrix(mode):
    outs = run_ranks("collective_worker.py", _ranks(), [mode], timeout=600)
    assert all(f"{mode} ok" in o for o in outs), outs
