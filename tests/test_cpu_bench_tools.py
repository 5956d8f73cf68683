"""Host-side logic of the benchmark tools (no GPU)."""
from nano_nccl_b200.bench.fused_trace import digest
from nano_nccl_b200.bench.variant_sweep import parse_variants


def test_trace_digest_separates_waiting_for_mma_from_draining():
    trace = {
        0: {"epilogue": [(0, 1000), (1, 5000), (3, 9000), (4, 9500), (1, 12000), (2, 15000), (3, 16000)],
            "producer": [(5, 2000), (6, 4000)]},
        1: {"epilogue": [(0, 1100), (1, 6000), (3, 8000)]},
    }
    d = digest(trace)
    assert d["ctas"] == 2 and d["span_us"] == 15.0
    assert d["mma_wait_us"] == (7000 + 4900) / 2 / 1e3      # entry -> ready, handed back -> next ready
    assert d["drain_us"] == (8000 + 2000) / 2 / 1e3         # ready -> handed back
    assert d["peer_wait_us"] == (3000 + 0) / 2 / 1e3        # ready -> partials arrived (own tiles only)
    assert d["block_wait_us"] == 2.0 and d["block_wait_max_us"] == 2.0


def test_variant_parser():
    v = parse_variants("default; NANO_NCCL_TILE_BYTES=131072 ;NANO_NCCL_SKEW=1,NANO_NCCL_MAX_CTAS=64;")
    assert v[0] == ("default", {})
    assert v[1] == ("NANO_NCCL_TILE_BYTES=131072", {"NANO_NCCL_TILE_BYTES": "131072"})
    assert v[2][1] == {"NANO_NCCL_SKEW": "1", "NANO_NCCL_MAX_CTAS": "64"}


def test_tuner_rules_from_sweep_rows():
    from nano_nccl_b200.bench.emit_tuner_rules import choose, merge, render

    def row(nbytes, algo, grid, us, dtype="bf16", coll="all_reduce", n=8):
        return {"collective": coll, "dtype": dtype, "op": "sum", "bytes": nbytes, "impl": "nano", "algo": algo,
                "grid": grid, "nranks": n, "p50_us": us}

    rows = []
    for dtype in ("bf16", "float"):
        rows += [row(1 << 18, "oneshot", 16, 20.0, dtype), row(1 << 18, "oneshot", 128, 20.1, dtype),   # tie: smaller grid
                 row(1 << 18, "twoshot", 128, 30.0, dtype),
                 row(1 << 20, "oneshot", 16, 25.0, dtype), row(1 << 20, "twoshot", 128, 31.0, dtype),
                 row(1 << 24, "oneshot", 16, 300.0, dtype), row(1 << 24, "twoshot", 128, 80.0, dtype)]
    rows.append({"collective": "all_reduce", "dtype": "bf16", "op": "sum", "bytes": 1 << 24, "impl": "nccl", "algo": "nccl",
                 "grid": 0, "nranks": 8, "p50_us": 1.0})                                               # ignored
    rules = merge(choose(rows))
    assert rules == [("all_reduce", 8, 1 << 22, "oneshot", 16), ("all_reduce", 8, None, "twoshot", 128)]
    text = render(rules)
    assert "all_reduce 8 4194304 oneshot 16\n" in text and "all_reduce 8 inf twoshot 128\n" in text


def test_reference_comparison_parsers():
    """The two table formats the side-by-side runner reads: the reference's benchmark rows (printed by the
    reference's own binaries: algo dtype redop transport size count time algbw busbw wrong max_abs) and this
    library's rows (collective dtype op algo bytes count host_us dev_p50 dev_avg algbw busbw wrong max_abs)."""
    from baseline.compare_reference import parse_nano, parse_reference

    ref_out = "\n".join([
        "# nano-nccl one-process-per-GPU all_reduce_bench",
        "#           algo    dtype    redop  transport      size(B)        count   time(us)      algbw      busbw    wrong      max_abs",
        "    ring_simple    float      sum        p2p       262144        65536      51.26       5.11       5.11        0            0",
        "    ring_simple    float      sum        p2p     67108864     16777216    2511.47      26.72      26.72        0            0",
        "rank=0 note: something unrelated",
    ])
    ref = parse_reference(ref_out)
    assert set(ref) == {262144, 67108864}
    assert ref[67108864] == {"time_us": 2511.47, "busbw": 26.72, "wrong": 0, "transport": "p2p"}
    nano_out = "\n".join([
        "# timing=host_wall+device_events wait_mode=query rank_aggregation=max warmup=5 iters=20",
        "collective     dtype op   algo          bytes        count    host_us  dev_p50us  dev_avgus     algbw     busbw  wrong  max_abs",
        "all_reduce     float sum  oneshot       262144        65536      27.81      19.94      19.88     13.15     13.15      0        0",
        "all_reduce     float sum  twoshot     67108864     16777216     182.32     173.92     173.57    385.86    385.86      0        0",
        "# diag rank=0 bytes=262144 enqueue_max_us=9.7 wait_max_us=24.0 host_us=27.8",
    ])
    nano = parse_nano(nano_out)
    assert set(nano) == {262144, 67108864}
    assert nano[67108864] == {"time_us": 182.32, "dev_p50_us": 173.92, "busbw": 385.86, "wrong": 0, "algo": "twoshot"}


def test_performance_matrix_renderer():
    from nano_nccl_b200.bench.render_performance import render

    def row(impl, algo, us, nbytes=1 << 20, coll="all_reduce", n=8):
        return {"collective": coll, "dtype": "bf16", "op": "sum", "bytes": nbytes, "impl": impl, "algo": algo, "grid": 0,
                "nranks": n, "p50_us": us, "min_us": us, "algbw_gbs": nbytes / us / 1e3, "busbw_gbs": nbytes / us / 1e3 * 1.75}

    rows = [row("nano", "oneshot", 30.0), row("nano", "twoshot", 25.0), row("nccl", "nccl", 40.0),
            row("nano", "nvls_symmetric_inplace", 20.0),                      # reported apart, never the cell's "nano"
            row("nano", "twoshot", 200.0, 1 << 26), row("nccl", "nccl", 100.0, 1 << 26)]
    text = render(rows)
    assert "## 8 GPUs" in text
    assert "| all_reduce | bf16 | sum | 1 MiB | twoshot | 25.00 | 40.00 |" in text        # the best non-symmetric algorithm
    assert "1.600" in text and "0.500" in text                                           # NCCL time / nano time per cell
    assert "geomean NCCL time / nano time = **0.894** over 2 cells" in text               # sqrt(1.6 * 0.5)
    assert "nano faster in 1 of 2" in text


def test_clock_sampler_summary():
    from nano_nccl_b200.utils.timing import ClockSampler

    s = ClockSampler()
    s.lines = ["0, 1965, 1965, 712.31, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
               "0, 1860, 1965, 998.10, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
               "0, 1920, 1965, 990.00, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active",
               "garbage line", "0, [N/A], 1965, 1, 0, Not Active, Not Active, Not Active, Not Active"]
    out = s.stop()
    assert out == {"sm_mhz": 1920.0, "sm_max_mhz": 1965.0, "samples": 3, "reasons": ["sw_power_cap"]}
    s2 = ClockSampler()
    s2.lines = ["0, 1200, 1965, 300, 0x8, Active, Not Active, Active, Not Active"]
    assert s2.stop()["reasons"] == ["hw_slowdown", "sw_thermal_slowdown"]


def test_trace_digest_times_the_flag_publisher_of_gemm_rs():
    """In GEMM->ReduceScatter the second time line of a CTA belongs to the flag publisher: tag 7 = a foreign
    tile's stores all issued, tag 4 = its flag published."""
    trace = {0: {"epilogue": [(0, 1000), (1, 5000), (3, 9000), (1, 12000), (3, 16000)],
                 "producer": [(7, 9100), (4, 12100), (7, 16200), (4, 18200)]}}
    d = digest(trace)
    assert d["publish_us"] == 5.0 and d["block_wait_us"] == 0.0
    assert d["span_us"] == 17.2


def test_headline_grid_summary_and_native_rows():
    from nano_nccl_b200.bench.headline import busbw_factor, parse_nano_bench, summarize

    assert busbw_factor("all_reduce", 8) == 2 * 7 / 8 and busbw_factor("all_gather", 2) == 0.5

    def cell(impl, coll, nbytes, us, bw):
        return {"collective": coll, "dtype": "bf16", "bytes": nbytes, "impl": impl, "p50_us": us, "busbw_gbs": bw}

    s = summarize([cell("nano", "all_reduce", 1 << 20, 10.0, 100.0), cell("nccl", "all_reduce", 1 << 20, 20.0, 50.0),
                   cell("nano", "all_gather", 1 << 20, 30.0, 40.0), cell("nccl", "all_gather", 1 << 20, 15.0, 80.0)])
    assert s["cells_compared"] == 2 and s["cells_faster_than_nccl"] == 1
    assert s["geomean_nccl_time_over_nano_time"] == 1.0          # 2.0 and 0.5
    assert s["cells_slower_than_nccl"] == [{"collective": "all_gather", "dtype": "bf16", "bytes": 1 << 20, "ratio": 0.5}]
    assert s["geomean_busbw_gbs"] == round((100.0 * 40.0) ** 0.5, 2)
    rows = parse_nano_bench("\n".join([
        "# header",
        "collective     dtype op   algo          bytes        count    host_us  dev_p50us  dev_avgus     algbw     busbw  wrong  max_abs",
        "all_reduce     float sum  oneshot       262144        65536      27.81      19.94      19.88     13.15     13.15      0        0",
    ]))
    assert rows == [{"collective": "all_reduce", "dtype": "float", "bytes": 262144, "algo": "oneshot", "host_us": 27.81,
                     "dev_p50_us": 19.94, "busbw_gbs": 13.15, "wrong": 0}]


def test_multi_gpu_rank_choice(monkeypatch):
    import conftest

    monkeypatch.setattr(conftest, "gpu_count", lambda: 8)
    monkeypatch.delenv("NANO_NCCL_TEST_RANKS", raising=False)
    assert conftest.multi_gpu_ranks() == 2
    monkeypatch.setenv("NANO_NCCL_TEST_RANKS", "8")
    assert conftest.multi_gpu_ranks() == 8 and conftest.multi_gpu_ranks(4) == 4
    monkeypatch.setenv("NANO_NCCL_TEST_RANKS", "4")
    assert conftest.multi_gpu_ranks() == 4
    monkeypatch.setattr(conftest, "gpu_count", lambda: 3)
    assert conftest.multi_gpu_ranks() == 2


def test_native_table_runs_the_native_programs_with_the_reference_arguments(tmp_path, monkeypatch):
    """`native_table` with a stand-in launcher and stand-in programs: arguments, host-loop bus bandwidth, notes."""
    import stat
    import sys

    from nano_nccl_b200.bench import headline

    log = tmp_path / "calls.log"
    launcher = tmp_path / "nano_nccl_mpirun"
    launcher.write_text("#!/bin/sh\nshift 4\nexec \"$@\"\n")
    row = "{coll}  {dtype} sum  oneshot  1048576  262144  50.00  40.00  41.00  20.97  {bw}  0  0"
    for name in ("nano_nccl_all_reduce_bench", "nano_nccl_collective_bench"):
        prog = tmp_path / name
        prog.write_text(f"#!{sys.executable}\nimport sys\nopen({str(log)!r}, 'a').write(' '.join(sys.argv[1:]) + '\\n')\n"
                        "a = sys.argv\ncoll = a[a.index('--collective') + 1]\ndtype = a[a.index('--dtype') + 1]\n"
                        f"print('# header line')\nprint({row!r}.format(coll=coll, dtype=dtype, bw='99.9'))\n"
                        "sys.exit(3 if coll == 'all_gather' and dtype == 'fp16' else 0)\n")
    for f in tmp_path.iterdir():
        f.chmod(f.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setattr(headline, "LIB", tmp_path)
    t = headline.native_table(4, budget_s=60)
    assert len(t["cells"]) == 9 and t["wrong_elements"] == 0
    ar = next(c for c in t["cells"] if c["collective"] == "all_reduce" and c["dtype"] == "bf16")
    assert ar["busbw_gbs"] == round(1048576 / 50.0 / 1e3 * 2 * 3 / 4, 2)     # from the host time, not the printed column
    ag = next(c for c in t["cells"] if c["collective"] == "all_gather" and c["dtype"] == "float")
    assert ag["busbw_gbs"] == round(1048576 / 50.0 / 1e3 * 3 / 4, 2)
    assert t["notes"] == ["all_gather/fp16: exit 3: # header line | all_gather  fp16 sum  oneshot  1048576  262144  50.00  40.00  41.00  20.97  99.9  0  0"]
    calls = log.read_text().splitlines()
    assert len(calls) == 9 and all(c.endswith("-b 262144 -e 67108864 -f 4 -w 5 -n 20") for c in calls)
    assert all(("--redop sum" in c) == ("all_gather" not in c) for c in calls)
    assert headline.native_table(4, budget_s=-1)["cells"] == []
