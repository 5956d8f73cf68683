"""Ring / Simple fallback path over each same-host transport, 2+ GPUs."""
import pytest

from _spawn import run_ranks
from conftest import multi_gpu_ranks

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("transport", ["p2p", "shm", "socket"])
def test_ring_fallback(transport):
    ranks = multi_gpu_ranks(4)
    env = {}
    if transport == "socket":
        # no network on the test machines: the loopback interface stands in for the NIC
        env = {"NANO_NCCL_SOCKET_IFNAME": "lo", "NANO_NCCL_SOCKET_ALLOW_LOOPBACK": "1"}
    outs = run_ranks("ring_worker.py", ranks, [transport], env=env, timeout=600)
    assert all(f"ring {transport} ok" in o for o in outs), outs
