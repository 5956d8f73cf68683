import pytest

from _spawn import run_ranks

pytestmark = pytest.mark.gpu


def test_single_rank_communicator():
    assert "single ok" in run_ranks("single_rank_worker.py", 1)[0]


def test_failed_drain_at_teardown_is_quarantined_by_default():
    out = run_ranks("teardown_policy_worker.py", 1, ["quarantine"])[0]
    assert "leaving its device memory mapped" in out and "teardown policy ok" in out, out


def test_failed_drain_at_teardown_ends_the_process_when_asked():
    with pytest.raises(AssertionError) as info:
        run_ranks("teardown_policy_worker.py", 1, ["abort"])
    text = str(info.value)
    assert "NANO_NCCL_TEARDOWN=abort: ending the process" in text and "teardown policy ok" not in text, text
