"""The sequence-parallel transformer block on the fused GEMM + collective kernels against the same block on
NCCL collectives, forward and backward, 2+ GPUs."""
import pytest

from _spawn import run_ranks
from conftest import multi_gpu_ranks

pytestmark = pytest.mark.gpu


def test_sequence_parallel_block_on_fused_kernels():
    ranks = multi_gpu_ranks()
    outs = run_ranks("tp_gpu_worker.py", ranks, timeout=300)
    assert all("tp gpu ok" in o for o in outs), outs
