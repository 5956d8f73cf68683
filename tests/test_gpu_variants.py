"""Kernel variants behind environment switches, on ONE GPU (emulated ranks where ranks are needed)."""
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

WORKER = Path(__file__).resolve().parent / "workers" / "variant_checks.py"


@pytest.mark.parametrize("case", ["bulk_copy", "emu_tma_allgather", "emu_ll", "fused_single", "emu_pipe"])
def test_variant(case):
    p = subprocess.run([sys.executable, str(WORKER), case], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and f"{case} ok" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.parametrize("depth", [1, 2, 8])
def test_pipelined_kernels_at_other_depths(depth):
    import os

    env = dict(os.environ, NANO_TEST_PIPE_DEPTH=str(depth))
    p = subprocess.run([sys.executable, str(WORKER), "emu_pipe"], capture_output=True, text=True, timeout=900, env=env)
    assert p.returncode == 0 and "emu_pipe ok" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]
