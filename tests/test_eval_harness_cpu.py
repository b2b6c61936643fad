"""Generate/build/run/compare harness: prompts, provider routing (fake HTTP), platform detection
(fake tools), the compile-and-run core and the round loop with a scripted "model"."""
import json
import os
import shutil
import sys

import pytest

from commbench_b200.harness import compile_run as CR
from commbench_b200.harness import eval_driver as ED
from commbench_b200.harness import platform_detect as PD
from commbench_b200.harness import task_runner as TR
from commbench_b200.harness.llm import factory as F
from commbench_b200.harness.llm import prompt as P

TASKS = os.path.join(os.path.dirname(CR.__file__), "tasks")


# ------------------------------------------------------------------------------- prompts
def test_code_extraction_variants():
    assert P.extract_code_from_response("text\n```python\nprint(1)\n```\nbye", "python") == "print(1)\n"
    two = "```text\nnote\n```\n```cuda\n__global__ void k(){}\nint main(){}\n```"
    assert "__global__" in P.extract_code_from_response(two, "cuda")
    cut = "Here it is:\n```cpp\nint main() {\n  return 0;"
    assert P.extract_code_from_response(cut, "cpp").startswith("int main()")
    assert P.extract_code_from_response("int x;", "cpp") == "int x;\n"
    assert P.extract_code_from_response("", "cpp") == ""


def test_prompts_carry_rules_history_and_caps(tmp_path):
    sk = tmp_path / "empty_x.cu"
    sk.write_text("// TODO\nint main(){return 0;}\n")
    c = P.generate_completion_prompt(str(sk), "Do the thing.")
    assert "sm_100a" in c and "Do the thing." in c and "```cuda" in c and "bounded" in c
    hist = [{"code": f"int main(){{return {i};}}\n", "error": "E" * 5000} for i in range(4)]
    f = P.generate_fix_prompt_from_code(str(sk), "int main(){}", "boom " * 1000, hist)
    assert f.count("Earlier attempt") == P.MAX_HISTORY and "Earlier attempt 3" in f and "Earlier attempt 4" in f
    assert "characters omitted" in f and "```diff" in f
    assert len(f) < 4 * (P.MAX_DIFF_CHARS + P.MAX_ERROR_CHARS)
    pf = P.generate_perf_fix_prompt_from_code(str(sk), "int main(){}", {"performance": "degraded"})
    assert "degraded" in pf and "faster" in pf
    py = tmp_path / "empty_y.py"
    py.write_text("# TODO\n")
    assert "127.0.0.1" in P.generate_completion_prompt(str(py))


# ------------------------------------------------------------------------------- factory
def test_provider_routing_and_model_lists():
    assert F.provider_for_model("gpt-4o") is F.Provider.OPENAI
    assert F.provider_for_model("o3-mini") is F.Provider.OPENAI
    assert F.provider_for_model("claude-opus-4-5") is F.Provider.ANTHROPIC
    assert F.provider_for_model("gemini-2.5-pro") is F.Provider.GEMINI
    assert F.provider_for_model("grok-4") is F.Provider.GROK
    assert F.provider_for_model("deepseek-reasoner") is F.Provider.DEEPSEEK
    assert F.provider_for_model("z-ai/glm-4.6") is F.Provider.GLM
    assert F.provider_for_model("qwen3-coder-plus") is F.Provider.QWEN
    assert F.provider_for_model("kimi-k2-thinking") is F.Provider.MOONSHOT
    with pytest.raises(F.LLMError):
        F.provider_for_model("llama-3")
    assert set(F.list_supported_models()) == {p.value for p in F.Provider}


def test_request_quirks_per_provider():
    S = F.SPECS
    _, h, b = F.build_request(S[F.Provider.OPENAI], "gpt-4o", "p", 0.3, "k")
    assert b["temperature"] == 0.3 and h["Authorization"] == "Bearer k"
    _, _, b = F.build_request(S[F.Provider.OPENAI], "o1-mini", "p", 0.3, "k")
    assert "temperature" not in b and "max_completion_tokens" in b
    _, _, b = F.build_request(S[F.Provider.DEEPSEEK], "deepseek-reasoner", "p", 0.3, "k")
    assert "temperature" not in b
    _, _, b = F.build_request(S[F.Provider.MOONSHOT], "kimi-k2-0905-preview", "p", 0.2, "k")
    assert b["temperature"] == 1.0
    _, _, b = F.build_request(S[F.Provider.QWEN], "qwen3-max", "p", 0.2, "k")
    assert b["enable_thinking"] is False
    u, h, b = F.build_request(S[F.Provider.ANTHROPIC], "claude-opus-4-5", "p", 0.2, "k")
    assert h["x-api-key"] == "k" and b["system"] == F.SYSTEM_MESSAGE and "anthropic-version" in h
    u, _, b = F.build_request(S[F.Provider.GEMINI], "gemini-2.5-pro", "p", 0.2, "k")
    assert "gemini-2.5-pro:generateContent?key=k" in u and b["generationConfig"]["temperature"] == 0.2


def test_generate_code_with_fake_transport_and_retries(monkeypatch):
    monkeypatch.setenv("OPENAI_API_KEY", "test-key")
    calls, sleeps = [], []

    def flaky(url, headers, body, timeout):
        calls.append(body["model"])
        if len(calls) < 3:
            raise F.LLMError("HTTP 429", 429, True)
        return {"choices": [{"message": {"content": "```cuda\nint main(){}\n```"}}]}

    code = F.generate_code("p", "gpt-4o", "cuda", transport=flaky, sleep=sleeps.append)
    assert code == "int main(){}\n" and len(calls) == 3 and len(sleeps) == 2 and sleeps[1] > sleeps[0] - 2.0

    def fatal(*a):
        raise F.LLMError("HTTP 401", 401, False)

    with pytest.raises(F.LLMError):
        F.generate_code("p", "gpt-4o", transport=fatal, sleep=sleeps.append)
    monkeypatch.delenv("ANTHROPIC_API_KEY", raising=False)
    with pytest.raises(F.LLMError, match="ANTHROPIC_API_KEY"):
        F.generate_code("p", "claude-opus-4-5", transport=fatal)
    ok = F.generate_response("p", "claude-opus-4-5", api_key="k",
                             transport=lambda *a: {"content": [{"type": "text", "text": "hi"}]})
    assert ok == "hi"
    assert 2.0 <= F.backoff_delay(0, rng=lambda: 0.0) <= 4.0 and F.backoff_delay(10) == 60.0


# ---------------------------------------------------------------------- platform detection
_TOPO = """\tGPU0\tGPU1\tGPU2\tGPU3\tCPU Affinity
GPU0\t X \tNV18\tNV18\tNV18\t0-31
GPU1\tNV18\t X \tNV18\tNV18\t0-31
GPU2\tNV18\tNV18\t X \tNV18\t0-31
GPU3\tNV18\tNV18\tNV18\t X \t0-31
"""


def test_platform_detection_with_fake_tools(tmp_path):
    def runner(cmd):
        if cmd[0].endswith("nvcc"):
            return True, "Cuda compilation tools, release 12.9, V12.9.86"
        if "--query-gpu=name,driver_version,compute_cap,memory.total" in cmd:
            return True, "\n".join(["NVIDIA B200, 580.159, 10.0, 183359"] * 4)
        if cmd[1:3] == ["topo", "-m"]:
            return True, _TOPO
        return False, ""

    which = lambda n: {"nvcc": "/x/nvcc", "nvidia-smi": "/x/nvidia-smi"}.get(n)
    info = PD.detect_platform(runner, which)
    assert info.gpu.count == 4 and info.gpu.is_blackwell_dc and info.gpu.nvcc_version == "12.9"
    assert info.gpu.nvlink_peers == 3 and info.gpu.nvswitch is True
    assert info.platform_string().startswith("B200_NVLINK")
    assert json.loads(json.dumps(info.to_dict()))["gpu"]["count"] == 4
    none = PD.detect_platform(lambda c: (False, ""), lambda n: None)
    assert none.platform_string().startswith("CPU") and not none.gpu.available
    sys_ib = tmp_path / "infiniband" / "mlx5_0" / "ports" / "1"
    sys_ib.mkdir(parents=True)
    (sys_ib / "link_layer").write_text("Ethernet\n")
    net = PD.detect_network(lambda c: (False, ""), lambda n: None, sysfs=str(tmp_path / "infiniband"))
    assert net.kind == "roce" and net.devices == ["mlx5_0"]
    assert PD.parse_topology("") == (0, None)


# ------------------------------------------------------------------------ compile and run
def test_first_json_and_metrics_parsing():
    out = 'log {not json}\n{"Correctness": "PASS", "metrics": [{"data_size": 1, "latency_avg": 2.0}]} tail'
    j = CR.first_json_object(out)
    assert j["Correctness"] == "PASS" and CR.metrics_average(j)["latency_avg"] == 2.0
    assert CR.extract_metrics('x\nMETRICS_JSON: {"throughput_gbps": 0.85}\n') == {"throughput_gbps": 0.85}
    assert CR.first_json_object("nothing") is None
    env = CR.scrubbed_env({"A": 1})
    assert env["A"] == "1" and "TORCH_CUDA_ARCH_LIST" not in env and CR.REPO_ROOT in env["PYTHONPATH"]


def _python_task(tmp_path, body_ok=True):
    t = tmp_path / "toy"
    t.mkdir()
    (t / "task.json").write_text(json.dumps({"name": "toy", "launcher": "python", "timeout_s": 60,
                                             "primary_metric": "latency_avg", "direction": "lower"}))
    prog = ('import json\nprint(json.dumps({"Correctness": "%s", "metrics": '
            '[{"data_size": 1, "latency_avg": %f}]}))\n')
    (t / "empty_toy.py").write_text("# TODO: print the result JSON\nraise NotImplementedError\n")
    (t / "ref_toy.py").write_text(prog % ("PASS", 10.0))
    return t, prog


def test_compile_and_run_analysis(tmp_path):
    t, prog = _python_task(tmp_path)
    good = t / "cand.py"
    good.write_text(prog % ("PASS", 5.0))
    r = CR.compile_and_run(str(t), str(good))
    assert r.compile_success and r.run_success and CR.analyze_result(r)[0]
    bad = t / "bad.py"
    bad.write_text("def broken(:\n")
    r = CR.compile_and_run(str(t), str(bad))
    assert not r.compile_success and "Build error" in CR.get_error_details(r)
    fail = t / "fail.py"
    fail.write_text(prog % ("FAIL", 5.0))
    assert CR.analyze_result(CR.compile_and_run(str(t), str(fail))) == (False, "program reported FAIL")
    hang = t / "hang.py"
    hang.write_text("import time\ntime.sleep(60)\n")
    r = CR.compile_and_run(str(t), str(hang), timeout_s=1.5)
    assert r.timed_out and CR.analyze_result(r) == (False, "run timed out")
    s = TR.compare(str(t), str(t / "ref_toy.py"), str(good), str(tmp_path / "res"), plot=True)
    assert s["performance"] == "better" and s["performance_detail"]["improvement_pct"] == 50.0
    assert os.path.exists(tmp_path / "res" / "gen_metrics.csv") and os.path.exists(tmp_path / "res" / "summary.json")


# ----------------------------------------------------------------------------- round loop
def test_round_loop_repairs_then_tunes(tmp_path):
    t, prog = _python_task(tmp_path)
    replies = ["def broken(:\n", prog % ("PASS", 30.0), prog % ("PASS", 9.8)]
    prompts = []

    def model(prompt, model_name, language, temperature):
        prompts.append(prompt)
        return replies[len(prompts) - 1]

    passed, reason, result, rounds, perf = ED.generate_eval_one(
        str(t), "fake-model", max_rounds=4, generate=model, quiet=True)
    assert passed and rounds == 3 and perf["performance"] == "on_par"
    assert "Complete every part marked TODO" in prompts[0]
    assert "failed. Fix it." in prompts[1] and "Build error" in prompts[1]
    assert "slower than the reference" in prompts[2] and "severely_degraded" in prompts[2]
    final = json.load(open(t / "results" / "fake-model" / "summary.json"))
    assert final["pass_iteration"] == 2 and final["improvement_iteration"] == 3 and final["model"] == "fake-model"
    rdirs = sorted(os.listdir(t / "results" / "fake-model"))
    assert sum(d.startswith("round") for d in rdirs) == 3
    assert os.path.exists(t / "results" / "fake-model" / rdirs[0] / "prompt.txt")
    # a correct candidate whose reference prints no primary metric is judged
    # "no_baseline_metrics": accepted at once (no tuning round), and it counts as passed
    (t / "ref_toy.py").write_text('import json\nprint(json.dumps({"Correctness": "PASS", "metrics": []}))\n')
    asked = []

    def once(prompt, *a):
        asked.append(prompt)
        return prog % ("PASS", 30.0)

    passed, reason, result, rounds, perf = ED.generate_eval_one(
        str(t), "m3", max_rounds=4, generate=once, quiet=True)
    assert passed and rounds == 1 and len(asked) == 1
    assert perf["performance"] == "no_baseline_metrics"
    assert ED.ACCEPTABLE is __import__("commbench_b200.harness.verdict", fromlist=["x"]).ACCEPTABLE
    (t / "ref_toy.py").write_text(prog % ("PASS", 10.0))
    # never passes: gives up after max_rounds with the last reason
    passed, reason, *_ = ED.generate_eval_one(str(t), "m2", max_rounds=2, quiet=True,
                                              generate=lambda *a: "raise SystemExit(3)\n")
    assert not passed and "run failed" in reason


def test_transient_model_errors_are_retried():
    n, sleeps = [0], []

    def flaky():
        n[0] += 1
        if n[0] < 3:
            raise TimeoutError("request timed out")
        return "ok"

    assert ED.call_with_retry(flaky, sleep=sleeps.append) == "ok" and len(sleeps) == 2
    with pytest.raises(ValueError):
        ED.call_with_retry(lambda: (_ for _ in ()).throw(ValueError("bad")), sleep=sleeps.append)


@pytest.mark.slow
@pytest.mark.timeout(300)
def test_shipped_gloo_task_reference_passes_its_own_check():
    """The shipped all-reduce task: the reference file, run as a candidate on two gloo ranks."""
    folder = os.path.join(TASKS, "gloo_allreduce")
    ref = CR.find_ref_file(folder)
    assert CR.find_empty_file(folder).endswith("empty_gloo_allreduce.py") and ref
    r = CR.compile_and_run(folder, ref, work_dir="/tmp/cb_task_build")
    assert CR.analyze_result(r) == (True, "program reported PASS"), r.output[-2000:]
    assert CR.metrics_average(r.result_json)["data_size_avg"] == 4.0
    skel = CR.compile_and_run(folder, CR.find_empty_file(folder), work_dir="/tmp/cb_task_build")
    assert not CR.analyze_result(skel)[0]            # the unfilled skeleton must not pass
    shutil.rmtree("/tmp/cb_task_build", ignore_errors=True)


def test_leaderboard_scoring_and_table(tmp_path):
    from commbench_b200.harness import leaderboard as LB

    def summ(task, model, pass_it, perf, base=None, cand=None, direction="lower"):
        d = tmp_path / task / "results" / model
        d.mkdir(parents=True)
        detail = {"primary_metric": "latency_avg", "direction": direction, "baseline": base, "candidate": cand}
        (d / "summary.json").write_text(json.dumps(
            {"task": task, "model": model, "passed": pass_it is not None and perf in ("better", "on_par"),
             "pass_iteration": pass_it, "performance": perf, "performance_detail": detail}))

    summ("t1", "m-a", 1, "better", 100.0, 50.0)                   # 2x faster (lower is better)
    summ("t2", "m-a", 2, "degraded", 10.0, 20.0, "lower")         # 0.5x
    summ("t3", "m-a", None, None)
    summ("t1", "m-b", 1, "on_par", 4.0, 4.0, "higher")
    table = LB.score(LB.collect(str(tmp_path)))
    a, b = table["m-a"], table["m-b"]
    assert a["tasks"] == 3 and a["correct"] == 2 and abs(a["pass_rate"] - 2 / 3) < 1e-9
    assert abs(a["pass_good_rate"] - 1 / 3) < 1e-9 and abs(a["gm_speedup"] - 1.0) < 1e-9
    assert abs(a["pass_x_gm"] - 2 / 3) < 1e-9 and a["mean_rounds_to_pass"] == 1.5
    assert b["pass_rate"] == 1.0 and b["gm_speedup"] == 1.0
    md = LB.render_markdown(table)
    assert md.splitlines()[2].startswith("| m-b |") and "| m-a | 3 | 67 % | 33 % | 1.00 | 0.67 | 1.5 |" in md


@pytest.mark.timeout(600)
def test_leaderboard_self_check_runs_references_as_candidates(tmp_path):
    """Copies two quick tasks, evaluates each reference as the candidate through the whole
    build / run / compare path and aggregates the result."""
    from commbench_b200.harness import leaderboard as LB

    for t in ("rdma_atomics", "rdma_memory_pool"):
        shutil.copytree(os.path.join(TASKS, t), tmp_path / t, ignore=shutil.ignore_patterns("results", "build"))
    rows = LB.run_all("reference", str(tmp_path), None, 1, self_check=True, log=lambda *_: None)
    assert [r["task"] for r in rows] == ["rdma_atomics", "rdma_memory_pool"]
    assert all(r["rounds"] == 1 and r["performance"] is not None for r in rows), rows
    table = LB.score(LB.collect(str(tmp_path)))
    assert table["reference"]["tasks"] == 2 and table["reference"]["correct"] == 2
    assert 0.2 < table["reference"]["gm_speedup"] < 5.0           # the same program twice
    assert LB.main(["--tasks-dir", str(tmp_path), "--out", str(tmp_path / "lb.md")]) == 0
    assert (tmp_path / "lb.json").exists() and "reference" in (tmp_path / "lb.md").read_text()


@pytest.mark.timeout(300)
def test_comparison_summary_has_the_documented_layout(tmp_path):
    """A real reference-vs-candidate comparison writes exactly the keys of the shipped template."""
    folder = os.path.join(TASKS, "rdma_memory_pool")
    ref = CR.find_ref_file(folder)
    s = CR.compare_save_results(folder, ref, ref, str(tmp_path / "cmp"))
    with open(os.path.join(os.path.dirname(CR.__file__), "summary_template.json")) as f:
        tmpl = json.load(f)
    assert set(s) == set(tmpl)
    assert set(s["build_and_run"]["generated"]) == set(tmpl["build_and_run"]["generated"])
    assert set(s["performance_detail"]) >= {"primary_metric", "direction", "baseline", "candidate",
                                            "improvement_pct"}
    assert s["latency_unit"] == "us" and s["ref_source"] == "ref_rdma_memory_pool.py"
    assert s["correctness"] == {"reference": True, "generated": True, "reason": "program reported PASS"}
    with open(tmp_path / "cmp" / "summary.json") as f:
        assert json.load(f)["task"] == "rdma_memory_pool"


@pytest.mark.timeout(300)
def test_relative_paths_survive_the_change_of_working_directory(tmp_path, monkeypatch):
    """Programs run with the task folder as their working directory; a relative task folder,
    source or build directory given by the caller must still mean what it meant for the caller."""
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    monkeypatch.chdir(repo)
    rel_task = os.path.relpath(os.path.join(TASKS, "rdma_atomics"), repo)
    rel_src = os.path.join(rel_task, "ref_rdma_atomics.py")
    work = os.path.relpath(str(tmp_path / "b"), repo)
    r = CR.compile_and_run(rel_task, rel_src, work_dir=work)
    assert CR.analyze_result(r) == (True, "program reported PASS"), r.output[-1500:]
    assert os.path.isabs(r.source)
    out = tmp_path / "tr"
    rc = TR.main(["--task", rel_task, "--compare", rel_src, rel_src, "--results-dir", str(out), "--plot"])
    assert rc == 0 and (out / "summary.json").exists() and (out / "latency.svg").exists()


def test_task_files_are_found_in_platform_subfolders(tmp_path):
    assert CR.platform_subdir_order("NV_ROCE")[:3] == ["", "nv", "roce"]
    assert CR.platform_subdir_order("CPU") == ["", "nv", "ib", "roce", "efa"]
    t = tmp_path / "task"
    (t / "nv").mkdir(parents=True)
    (t / "efa").mkdir()
    (t / "ib").mkdir()
    (t / "efa" / "empty_x.py").write_text("# efa\n")
    (t / "ib" / "empty_x.py").write_text("# ib\n")
    (t / "ib" / "ref_x.py").write_text("# ib\n")
    assert CR.find_empty_file(str(t), "NV_EFA").endswith(os.path.join("efa", "empty_x.py"))
    assert CR.find_empty_file(str(t), "NV_IB").endswith(os.path.join("ib", "empty_x.py"))
    assert CR.find_empty_file(str(t)).endswith(os.path.join("ib", "empty_x.py"))      # no NIC: ib first
    assert CR.find_ref_file(str(t), "NV_EFA").endswith(os.path.join("ib", "ref_x.py"))
    (t / "nv" / "empty_x.cu").write_text("// nv\n")
    assert CR.find_empty_file(str(t), "NV_EFA").endswith(os.path.join("nv", "empty_x.cu"))
    (t / "empty_x.py").write_text("# top\n")
    assert CR.find_empty_file(str(t), "NV_EFA") == str(t / "empty_x.py")              # the folder itself wins
    assert CR.find_ref_file(str(tmp_path)) is None
