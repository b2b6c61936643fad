"""Roofline arithmetic and verdict tiers (pure functions, no GPU)."""
import json

import pytest

from commbench_b200.harness import roofline as RF
from commbench_b200.harness import verdict as V


def test_link_bytes_follow_the_collective_conventions():
    S = 1 << 30
    assert RF.nvlink_bytes("all_reduce", S, 8) == pytest.approx(2 * 7 / 8 * S)      # ring equivalent
    assert RF.nvlink_bytes("all_reduce", S, 8, nvls=True) == S                      # reduced in the switch
    for op in ("all_gather", "reduce_scatter", "all_to_all"):
        assert RF.nvlink_bytes(op, S, 4) == pytest.approx(0.75 * S)
    assert RF.nvlink_bytes("broadcast", S, 2) == S
    assert RF.nvlink_bytes("all_reduce", S, 1) == 0.0
    with pytest.raises(KeyError):
        RF.nvlink_bytes("gossip", S, 2)
    assert RF.allreduce_bus_factor(8) == pytest.approx(1.75) and RF.allreduce_bus_factor(1) == 1.0


def test_roofline_takes_the_slower_of_compute_and_link(tmp_path):
    peaks = RF.Peaks(1600.0, 1400.0, 6650.0, 770.0, "measured")
    flops = 2.0 * 8192 * 8192 * 3584
    link = RF.nvlink_bytes("all_gather", 8192 * 8192 * 2, 8)
    t_compute, t_link = flops / 1600e12 * 1e3, link / 770e9 * 1e3
    assert RF.roofline_ms(flops, link, peaks) == pytest.approx(max(t_compute, t_link))
    assert RF.roofline_ms(flops, 0, peaks, sustained=True) == pytest.approx(flops / 1400e12 * 1e3)
    assert RF.roofline_ms(0, link, peaks) == pytest.approx(t_link)
    assert RF.fraction(0.3, 0.4) == pytest.approx(0.75) and RF.fraction(0.3, 0) is None
    # measured peaks file wins over the fall-back, and says so
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps(
        {"bf16_tflops": 1646.6, "bf16_tflops_sustained": 1383.9, "hbm_gbs": 6700.0}))
    p = RF.load_peaks(str(tmp_path))
    assert (p.bf16_tflops, p.bf16_tflops_sustained, p.source) == (1646.6, 1383.9, "measured")
    q = RF.load_peaks(str(tmp_path / "nowhere"))
    assert q.source == "fallback" and q.bf16_tflops == 1590.0 and q.nvlink_gbs == 770.0


def test_verdict_tiers_and_guards():
    lower = {"primary": "latency_avg", "direction": "lower"}
    higher = {"primary": "throughput_avg", "direction": "higher"}
    v = V.compute_verdict(lower, {"latency_avg": 100.0}, {"latency_avg": 79.0})
    assert v.verdict == "better" and v.detail["improvement_pct"] == 21.0 and v.acceptable
    assert V.compute_verdict(lower, {"latency_avg": 100.0}, {"latency_avg": 104.0}).verdict == "on_par"
    assert V.compute_verdict(lower, {"latency_avg": 100.0}, {"latency_avg": 130.0}).verdict == "degraded"
    sev = V.compute_verdict(lower, {"latency_avg": 100.0}, {"latency_avg": 150.0})
    assert sev.verdict == "severely_degraded" and not sev.acceptable
    assert V.compute_verdict(higher, {"throughput_avg": 10.0}, {"throughput_avg": 12.0}).verdict == "better"
    assert V.compute_verdict(higher, {"throughput_avg": 10.0}, {"throughput_avg": 5.9}).verdict == "severely_degraded"
    # a time of zero against a positive baseline was not measured
    z = V.compute_verdict(lower, {"latency_avg": 5.0}, {"latency_avg": 0.0})
    assert z.verdict == "severely_degraded" and "did-not-measure" in z.detail["note"]
    assert V.compute_verdict("info_only", {}, {}).verdict == "info_only"
    assert V.compute_verdict(lower, {"latency_avg": 1.0}, {}).verdict == "no_candidate_metrics"
    assert V.compute_verdict(lower, {}, {"latency_avg": 1.0}).verdict == "no_baseline_metrics"
    with pytest.raises(ValueError):
        V.improvement_pct(1.0, 1.0, "sideways")
    # values that are not numbers count as missing (candidate side first), a bad direction
    # gives "unknown" instead of an exception: a foreign summary must not crash a re-judge pass
    assert V.compute_verdict(lower, {"latency_avg": 1.0}, {"latency_avg": "N/A"}).verdict == "no_candidate_metrics"
    assert V.compute_verdict(lower, {"latency_avg": {"x": 1}}, {"latency_avg": 1.0}).verdict == "no_baseline_metrics"
    assert V.compute_verdict(lower, {"latency_avg": "N/A"}, {"latency_avg": True}).verdict == "no_candidate_metrics"
    odd = V.compute_verdict({"primary": "latency_avg", "direction": "sideways"},
                            {"latency_avg": 1.0}, {"latency_avg": 1.0})
    assert odd.verdict == "unknown" and odd.acceptable
    assert V.geometric_mean_speedup([(2.0, 1.0), (1.0, 2.0)]) == pytest.approx(1.0)
    assert V.geometric_mean_speedup([(3.0, 1.0)]) == pytest.approx(3.0)


def test_old_summaries_are_rejudged_and_keep_their_first_verdict(tmp_path):
    task = tmp_path / "some_task"
    res = task / "results" / "m" / "round1"
    res.mkdir(parents=True)
    (task / "task.json").write_text(json.dumps({"name": "some_task", "primary_metric": "throughput",
                                                "direction": "higher"}))
    # the older layout: two flat dicts and a two-word verdict
    p = res / "summary.json"
    p.write_text(json.dumps({"metrics_comparison": {"ref": {"throughput": 40.0, "latency_avg": 9.0},
                                                    "generated": {"throughput": 52.0, "latency_avg": 7.0}},
                             "performance": "same"}))
    assert V.infer_task_name(str(p)) == "some_task" and V.infer_task_name(str(res)) == "some_task"
    assert V.infer_task_name(str(tmp_path)) is None
    s = V.override_summary_verdict(str(p))
    assert s["performance"] == "better" and s["performance_legacy"] == "same"
    assert s["performance_detail"]["primary_metric"] == "throughput" and s["verdict_scheme"]["better_pct"] == 20.0
    again = V.override_summary_verdict(str(p), {"primary": "latency_avg", "direction": "lower"})
    assert again["performance"] == "better" and again["performance_legacy"] == "same"   # first verdict kept
    assert again["performance_detail"]["improvement_pct"] == pytest.approx(22.222, abs=1e-3)
    # the current layout, and a task without a metric of its own
    q = res / "s2.json"
    q.write_text(json.dumps({"metrics_comparison": {"latency_avg": {"reference": 10.0, "generated": 20.0}}}))
    assert V.override_summary_verdict(str(q), {"primary": "latency_avg", "direction": "lower"})["performance"] == \
        "severely_degraded"
    (task / "task.json").write_text(json.dumps({"name": "some_task"}))
    assert V.override_summary_verdict(str(q))["performance"] == "info_only"
