"""Test configuration: the `gpu` marker, an incremental native build, and helpers to run
multi-process cases (one process per GPU, or CPU-only ranks)."""
from __future__ import annotations

import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs at least one CUDA device (run on a B200)")


@pytest.fixture(scope="session", autouse=True)
def native_build():
    """Builds (incrementally) the native library and test programs once per session."""
    from nano_nccl_b200 import _build

    _build.build_programs(verbose=False)
    return _build


def gpu_count() -> int:
    try:
        import torch

        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


def multi_gpu_ranks(most: int = 8) -> int:
    """Rank count of a multi-GPU test: 2 by default, or the largest of 2 / 4 / 8 that fits the visible GPUs,
    `most` and NANO_NCCL_TEST_RANKS when that variable is set (one process per GPU).  Skips below 2 GPUs.
    The default stays at 2 because the host side of a test (reference results on the CPU, one interpreter per
    rank) grows with the rank count and a whole-suite run at 8 ranks takes many times longer."""
    n = gpu_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    want = int(os.environ.get("NANO_NCCL_TEST_RANKS", "2"))
    cap = min(n, most, max(want, 2))
    return 8 if cap >= 8 else 4 if cap >= 4 else 2
