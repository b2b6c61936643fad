"""Tracing helpers without a GPU: NVTX ranges are free no-ops, kernel-event aggregation, the
span recorder's Chrome trace."""
import json
import time

from commbench_b200.utils import tracing as TR


def test_nvtx_range_and_decorator_are_noops_without_cuda():
    calls = []

    @TR.traced("unit.fn")
    def fn(a, b=1):
        calls.append((a, b))
        return a + b

    with TR.nvtx_range("outer"):
        with TR.nvtx_range("inner", force=True):
            assert fn(2, b=3) == 5
    assert calls == [(2, 3)] and fn.__name__ == "fn"


def test_kernel_event_aggregation_by_name_and_by_substring():
    ev = [("cb::gemm_kernel<256>", 100.0), ("cb::gemm_kernel<256>", 140.0), ("cb::rs_kernel<0,8>", 30.0),
          ("elementwise_kernel", 5.0)]
    by_name = TR.aggregate_kernel_events(ev)
    assert by_name["cb::gemm_kernel<256>"] == {"calls": 2, "total_us": 240.0, "min_us": 100.0,
                                               "max_us": 140.0, "mean_us": 120.0}
    sel = TR.aggregate_kernel_events(ev, names=["gemm", "rs_kernel", "absent"])
    assert set(sel) == {"gemm", "rs_kernel"} and sel["rs_kernel"]["calls"] == 1
    assert sel["gemm"]["mean_us"] == 120.0


def test_kernel_times_runs_the_function_under_the_profiler():
    import torch

    n = []

    def fn():
        n.append(1)
        return torch.ones(64, 64) @ torch.ones(64, 64)

    out = TR.kernel_times(fn, iters=3, warmup=1)
    assert len(n) == 4 and out and all(v["calls"] >= 1 for v in out.values())


def test_span_recorder_nests_and_exports_a_chrome_trace(tmp_path):
    rec = TR.SpanRecorder(rank=3)
    with rec.span("step", index=0):
        with rec.span("dispatch"):
            time.sleep(0.002)
        with rec.span("gemm", tokens=128):
            time.sleep(0.001)
    rows = rec.spans()
    assert [r["name"] for r in rows] == ["step", "dispatch", "gemm"]
    assert [r["depth"] for r in rows] == [0, 1, 1]
    step, disp, gemm = rows
    assert step["dur_us"] >= disp["dur_us"] + gemm["dur_us"] and disp["dur_us"] >= 1500
    assert gemm["start_us"] >= disp["start_us"] + disp["dur_us"] - 1 and gemm["args"] == {"tokens": 128}
    p = rec.export(str(tmp_path / "trace" / "r3.json"))
    with open(p) as f:
        doc = json.load(f)
    xs = [e for e in doc["traceEvents"] if e["ph"] == "X"]
    assert len(xs) == 3 and all(e["pid"] == 3 for e in xs) and doc["traceEvents"][0]["ph"] == "M"
    rec2 = TR.SpanRecorder(rank=4)
    with rec2.span("other"):
        pass
    p2 = rec2.export(str(tmp_path / "trace" / "r4.json"))
    merged = TR.merge_chrome_traces([p, p2], str(tmp_path / "all.json"))
    with open(merged) as f:
        assert {e["pid"] for e in json.load(f)["traceEvents"]} == {3, 4}


def test_latency_stats_are_nearest_rank_percentiles():
    from commbench_b200.utils.timing import latency_stats

    s = latency_stats(range(1, 101))                  # 1 .. 100
    assert (s["count"], s["min"], s["max"], s["avg"]) == (100, 1.0, 100.0, 50.5)
    assert (s["p50"], s["p90"], s["p99"]) == (50.0, 90.0, 99.0)
    one = latency_stats([7.5])
    assert one["p50"] == one["p99"] == one["min"] == one["max"] == 7.5
    few = latency_stats([3.0, 1.0, 2.0])
    assert few["p50"] == 2.0 and few["p99"] == 3.0 and few["p90"] == 3.0
    assert latency_stats([])["count"] == 0 and latency_stats([])["p99"] is None
