"""Result store, suite-level resume, summary and stored reference points (no GPU)."""
import json
import os

from commbench_b200.harness import report


def _rec(op, variant, n, ms, base, world=2, **kw):
    return dict(key=report.config_key(op, variant, (n,), "bf16", world), op=op, variant=variant,
                shape=[n], dtype="bf16", world=world, correct=True, time_ms=ms, baseline_ms=base, **kw)


def test_store_survives_a_torn_line_and_overwrites_by_key(tmp_path):
    p = str(tmp_path / "r.jsonl")
    s = report.ResultStore(p)
    s.add(_rec("all_reduce", "nvls", 1024, 0.02, 0.03))
    s.add(_rec("all_reduce", "nvls", 1024, 0.01, 0.03))           # same key measured again
    with open(p, "a") as f:
        f.write('{"key": "broken", "op": ')                         # interrupted write
    s2 = report.ResultStore(p)
    assert len(s2.records()) == 1 and s2.records()[0]["time_ms"] == 0.01
    assert s2.has(report.config_key("all_reduce", "nvls", (1024,), "bf16", 2))


def test_suite_ledger_skips_only_when_every_rank_finished(tmp_path):
    stores = [report.ResultStore(str(tmp_path / f"rank{r}.jsonl")) for r in range(2)]
    params = {"quick": True, "scale": 1.0}
    votes = []

    def agree_with(other_flag):
        def agree(flag):
            votes.append(flag)
            return flag and other_flag
        return agree

    led0 = report.SuiteLedger(stores[0], 2, params, agree=agree_with(False))
    assert not led0.done("tp")
    led0.mark("tp")
    # rank 0 finished, rank 1 did not: both must run the suite again
    assert not report.SuiteLedger(stores[0], 2, params, agree=agree_with(False)).done("tp")
    assert report.SuiteLedger(stores[0], 2, params, agree=agree_with(True)).done("tp")
    # other arguments measure something else; resume off never skips; markers are not results
    assert not report.SuiteLedger(stores[0], 2, {"quick": False, "scale": 1.0}).done("tp")
    assert not report.SuiteLedger(stores[0], 2, params, enabled=False).done("tp")
    assert not report.SuiteLedger(stores[0], 4, params).done("tp")
    assert stores[0].records() == [] and votes[0] is False
    reopened = report.ResultStore(stores[0].path)
    assert report.SuiteLedger(reopened, 2, params).done("tp")


def test_summary_and_stored_reference_points(tmp_path):
    rows = [_rec("all_reduce", "nvls", 1 << 20, 0.020, 0.030, busbw_gbs=100.0, roofline_frac=0.2),
            _rec("all_reduce", "nvls", 1 << 10, 0.010, 0.009, busbw_gbs=1.0, roofline_frac=0.01),
            _rec("ag_gemm", "bf16", 4096, 0.4, 0.52, tflops=900.0, roofline_frac=0.8),
            {**_rec("barrier", "flag-matrix", 2, 0.003, None), "correct": True}]
    out = str(tmp_path / "out")
    s = report.write_summary(rows, out, meta={"world": 2})
    assert s["all_correct"] and len(s["entries"]) == 4
    verdicts = {(e["op"], e["shape"][0]): e["verdict"] for e in s["entries"]}
    assert verdicts[("all_reduce", 1 << 20)] == "better" and verdicts[("all_reduce", 1 << 10)] == "degraded"
    assert abs(s["geomean_speedup"] - (1.5 * 0.9 * 1.3) ** (1 / 3)) < 1e-9
    ref_dir = os.path.join(out, "performance_reference")
    names = sorted(os.listdir(ref_dir))
    assert names == ["ag_gemm_bf16_w2.json", "all_reduce_nvls_w2.json", "barrier_flag-matrix_w2.json"]
    with open(os.path.join(ref_dir, "all_reduce_nvls_w2.json")) as f:
        doc = json.load(f)
    assert doc["Correctness"] == "PASS" and doc["throughput_unit"] == "GB/s (bus)"
    assert [p["data_size"] for p in doc["metrics"]] == [1 << 10, 1 << 20]        # sorted by size
    assert doc["metrics"][1]["latency_avg"] == 20.0 and doc["metrics"][1]["baseline_latency_avg"] == 30.0
    with open(os.path.join(ref_dir, "ag_gemm_bf16_w2.json")) as f:
        assert json.load(f)["throughput_unit"] == "TFLOP/s"
    with open(os.path.join(out, "summary.csv")) as f:
        assert f.readline().startswith("op,variant,world")
