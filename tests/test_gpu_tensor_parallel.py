"""The sequence-parallel transformer block on the fused GEMM + collective kernels against the same block on
NCCL collectives, forward and backward, 2+ GPUs."""
import pytest

from _spawn import run_ranks
from conftest import gpu_count

pytestmark = pytest.mark.gpu


def test_sequence_parallel_block_on_fused_kernels():
    n = gpu_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    ranks = 8 if n >= 8 else 4 if n >= 4 else 2
    outs = run_ranks("tp_gpu_worker.py", ranks, timeout=300)
    assert all("tp gpu ok" in o for o in outs), outs
