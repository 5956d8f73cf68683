"""Host-side logic of the reference arm of bench.py, driven with stand-in programs (no GPU, no reference build):
which programs are launched with which arguments, how their tables are parsed, what is reported when a
program is missing, fails or the time budget runs out."""
import os
import stat
import sys

import pytest

from baseline import reference_arm

TABLE = """# nano-nccl one-process-per-GPU bench
#           algo    dtype    redop  transport      size(B)        count   time(us)      algbw      busbw    wrong      max_abs
    ring_simple    {dtype}      sum        p2p       262144        65536      50.00       5.24       5.24        0            0
    ring_simple    {dtype}      sum        p2p      1048576       262144     100.00      10.49      10.49        {wrong}            0
rank=0 note: not a row
"""


@pytest.fixture
def fake_tree(tmp_path, monkeypatch):
    """A launcher that runs the program it is given, and programs that print a reference-style table."""
    ref = tmp_path / "_ref"
    ref.mkdir()
    launcher = tmp_path / "mpirun"
    launcher.write_text("#!/bin/sh\n# usage: mpirun -np N --timeout T program args...\nshift 4\nexec \"$@\"\n")
    launcher.chmod(launcher.stat().st_mode | stat.S_IEXEC)
    log = tmp_path / "calls.log"

    def program(name: str, wrong: int = 0, exit_code: int = 0) -> None:
        body = (f"#!{sys.executable}\nimport sys\nopen({str(log)!r}, 'a').write(' '.join(sys.argv) + '\\n')\n"
                f"dtype = sys.argv[sys.argv.index('--dtype') + 1]\n"
                f"print({TABLE!r}.format(dtype=dtype, wrong={wrong}))\nsys.exit({exit_code})\n")
        path = ref / name
        path.write_text(body)
        path.chmod(path.stat().st_mode | stat.S_IEXEC)

    monkeypatch.setattr(reference_arm, "REF_DIR", ref)
    monkeypatch.setattr(reference_arm, "MPIRUN", launcher)
    return program, log


def test_reference_arm_runs_every_channel_count_and_parses_the_tables(fake_tree):
    program, log = fake_tree
    for c in (1, 2, 4):  # 3 channels: not built
        program(f"ref_all_reduce_bench_n2_c{c}")
        program(f"ref_collective_bench_n2_c{c}", wrong=3 if c == 1 else 0)
    out = reference_arm.run_reference(2, steps=5, warmup=3, budget_s=120)
    assert out["impl"] == "reference" and out["value"] is None and "unavailable" in out
    ch = out["collectives"]["channels"]
    assert list(ch) == ["4", "2", "1", "3"]                      # most important first
    assert len(ch["4"]["cells"]) == 3 * 3 * 2 and ch["4"]["wrong_elements"] == 0
    assert ch["1"]["wrong_elements"] == 3 * (2 * 3)              # 3 in one row of each collective-program launch: 2 collectives x 3 dtypes
    assert ch["3"]["cells"] == [] and all("is not built" in n for n in ch["3"]["notes"])
    cell = next(c for c in ch["4"]["cells"] if c["collective"] == "all_gather" and c["dtype"] == "bf16" and c["bytes"] == 1048576)
    assert cell["time_us"] == 100.0 and cell["busbw_gbs"] == round(1048576 / 100.0 / 1e3 * 0.5, 3)
    ar = next(c for c in ch["4"]["cells"] if c["collective"] == "all_reduce" and c["bytes"] == 262144)
    assert ar["busbw_gbs"] == round(262144 / 50.0 / 1e3 * 1.0, 3)  # 2 (N-1)/N at N = 2
    calls = log.read_text().splitlines()
    assert len(calls) == 3 * 9
    assert all("-b 262144 -e 67108864 -f 4 -w 5 -n 20" in c for c in calls)
    gathers = [c for c in calls if "--collective allgather" in c]
    assert gathers and all("--redop" not in c for c in gathers)  # the reference rejects an operator for AllGather
    assert all("--redop sum" in c for c in calls if "allgather" not in c)


def test_reference_arm_reports_failures_and_an_exhausted_budget(fake_tree):
    program, _ = fake_tree
    program("ref_all_reduce_bench_n4_c4", exit_code=7)
    program("ref_collective_bench_n4_c4")
    res = reference_arm.reference_collectives(4, budget_s=120)
    notes = res["channels"]["4"]["notes"]
    assert sum("exit 7" in n for n in notes) == 3                 # the three AllReduce dtypes; rows are still kept
    assert len(res["channels"]["4"]["cells"]) == 18
    res = reference_arm.reference_collectives(4, budget_s=-1.0)   # nothing may start
    assert all(e["cells"] == [] for e in res["channels"].values())
    assert all("time budget" in n for e in res["channels"].values() for n in e["notes"])
    assert res["best_geomean_busbw_gbs"] is None


def test_reference_arm_without_a_matching_build():
    out = reference_arm.run_reference(1, steps=1, warmup=1)
    assert "collectives" not in out and out["value"] is None
    out = reference_arm.run_reference(3, steps=1, warmup=1)
    assert "built: 2, 4, 8" in out["collectives"]["unavailable"]
