"""Communicator life-cycle cases on 2 GPUs: host-side fault injection with a fresh communicator afterwards, two
ranks on one device, two communicators with partial teardown (reference tests/mpi_transport_faults.cc,
tests/mpi_device_selection.cc, tests/mpi_c_api.cu).  Every failure is produced on the host before any kernel is
launched; multicast is off so that no rank leaves while its memory is bound to a multicast object."""
import pytest

from _spawn import run_ranks
from conftest import gpu_count

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["teardown", "same_device", "faults"])
def test_lifecycle(mode):
    if gpu_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    outs = run_ranks("lifecycle_worker.py", 2, [mode], env={"NANO_NCCL_NVLS": "0"}, timeout=300)
    assert all(f"{mode} ok" in o for o in outs), outs
