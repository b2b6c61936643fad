"""Every shipped generate/build/run task: well-formed description, skeleton and reference that
build, and - for the tasks that need no GPU - a reference that passes its own check while the
unfilled skeleton does not."""
import json
import os
import shutil

import pytest

from commbench_b200.harness import compile_run as CR

TASKS = os.path.join(os.path.dirname(CR.__file__), "tasks")
ALL = sorted(d for d in os.listdir(TASKS) if os.path.exists(os.path.join(TASKS, d, "task.json")))
CPU = [t for t in ALL if not CR.load_task(os.path.join(TASKS, t))["needs_gpu"]]
FAMILIES = {"A", "B", "C", "D", "E", "F", "G", "H", "I"}


def test_task_set_covers_several_families():
    fams = {CR.load_task(os.path.join(TASKS, t)).get("family") for t in ALL}
    assert len(ALL) >= 40 and {"A", "B", "C", "D", "F", "G", "H", "I"} <= fams
    assert fams <= FAMILIES | {None}


@pytest.mark.timeout(300)
@pytest.mark.parametrize("task", ["nvls_all_reduce", "ag_gemm_virtual_ranks"])
def test_gpu_task_skips_cleanly_without_enough_gpus(task, tmp_path):
    """A multi-GPU task launched on a machine that cannot run it prints Correctness SKIP and
    exits 0 before it creates a process group or a symmetric heap."""
    import torch

    folder = os.path.join(TASKS, task)
    spec = CR.load_task(folder)
    if torch.cuda.is_available() and torch.cuda.device_count() >= spec["world"]:
        pytest.skip("this machine can run the task")
    r = CR.compile_and_run(folder, CR.find_ref_file(folder), work_dir=str(tmp_path))
    assert r.run_success, r.output[-2000:]
    assert (r.result_json or {}).get("Correctness") == "SKIP"
    assert CR.analyze_result(r)[0]
    shutil.rmtree(os.path.join(folder, "__pycache__"), ignore_errors=True)


@pytest.mark.parametrize("task", ALL)
def test_task_is_well_formed(task):
    folder = os.path.join(TASKS, task)
    with open(os.path.join(folder, "task.json")) as f:
        spec = json.load(f)
    assert spec["name"] == task and len(spec["description"]) > 80
    assert spec["launcher"] in ("python", "torchrun", "nvcc") and spec["world"] >= 1
    assert spec["direction"] in ("lower", "higher") and spec["primary_metric"]
    empty, ref = CR.find_empty_file(folder), CR.find_ref_file(folder)
    assert empty and ref and os.path.splitext(empty)[1] == os.path.splitext(ref)[1]
    assert os.path.basename(empty) == "empty_" + os.path.basename(ref)[len("ref_"):]
    text = open(empty).read()
    assert "TODO" in text                                  # the skeleton says what to fill in
    assert (spec["launcher"] == "nvcc") == ref.endswith(".cu")


@pytest.mark.timeout(600)
@pytest.mark.parametrize("task", ALL)
def test_skeleton_and_reference_build(task, tmp_path):
    folder = os.path.join(TASKS, task)
    for src in (CR.find_ref_file(folder), CR.find_empty_file(folder)):
        r = CR.compile_and_run(folder, src, build_only=True, work_dir=str(tmp_path))
        assert r.compile_success, r.compile_output[-2000:]


@pytest.mark.slow
@pytest.mark.timeout(600)
@pytest.mark.parametrize("task", CPU)
def test_cpu_task_reference_passes_and_skeleton_does_not(task, tmp_path):
    """Reference and skeleton are launched side by side (separate work folders and rendezvous
    ports): most of a run is interpreter start-up of the ranks."""
    from concurrent.futures import ThreadPoolExecutor

    folder = os.path.join(TASKS, task)
    with ThreadPoolExecutor(2) as pool:
        f_ref = pool.submit(CR.compile_and_run, folder, CR.find_ref_file(folder),
                            work_dir=str(tmp_path / "ref"))
        f_skel = pool.submit(CR.compile_and_run, folder, CR.find_empty_file(folder),
                             work_dir=str(tmp_path / "skel"))
        r, skel = f_ref.result(), f_skel.result()
    assert CR.analyze_result(r) == (True, "program reported PASS"), r.output[-2000:]
    rows = (r.result_json or {}).get("metrics")
    spec = CR.load_task(folder)
    assert rows and all(spec["primary_metric"] in row for row in rows)
    assert not CR.analyze_result(skel)[0]
    shutil.rmtree(os.path.join(folder, "__pycache__"), ignore_errors=True)


def test_skeleton_generator_handles_markers_and_errors():
    from commbench_b200.harness import make_skeleton as MS

    ref = ('"""Doc.\n\nReference counterpart: somewhere\n(more).\n"""\n'
           "def f(x):\n    # --- solution: add one\n    #     (to x)\n    return x + 1\n    # --- end solution\n"
           "\n\ndef g():\n    # --- solution\n    return 2\n    # --- end solution\n")
    out = MS.skeleton_text(ref)
    assert "somewhere" not in out and "(more)" not in out and out.startswith('"""Doc.\n"""')
    assert "    # TODO: add one\n    #       (to x)\n    raise NotImplementedError\n" in out
    assert "    # TODO: implement\n    raise NotImplementedError\n" in out and "return" not in out
    cu = "bool w() {\n  // --- solution else: return false;: poll\n  return poll();\n  // --- end solution\n}\n"
    assert MS.skeleton_text(cu) == "bool w() {\n  // TODO: poll\n  return false;\n}\n"
    for bad in ("# --- end solution\n", "# --- solution: x\ncode\n",
                "# --- solution: a\n# --- solution: b\n# --- end solution\n"):
        with pytest.raises(ValueError):
            MS.skeleton_text(bad)
    assert MS.skeleton_path("/t/ref_x.py") == "/t/empty_x.py" and MS.has_markers(ref)


@pytest.mark.parametrize("task", ALL)
def test_marked_references_regenerate_their_committed_skeleton(task):
    from commbench_b200.harness import make_skeleton as MS

    ref = CR.find_ref_file(os.path.join(TASKS, task))
    text = open(ref).read()
    if not MS.has_markers(text):
        pytest.skip("skeleton of this task is kept by hand")
    assert open(MS.skeleton_path(ref)).read() == MS.skeleton_text(text)


@pytest.mark.timeout(600)
def test_cuda_build_reports_registers_and_is_cached(tmp_path):
    folder = os.path.join(TASKS, "mbarrier_producer_consumer")
    src = tmp_path / "ref_copy.cu"
    shutil.copy(CR.find_ref_file(folder), src)
    r1 = CR.compile_and_run(folder, str(src), build_only=True, work_dir=str(tmp_path / "b"))
    assert r1.compile_success and "[build cache hit]" not in r1.compile_output
    k = [p for p in r1.ptxas if "handoff_kernel" in p["kernel"]]
    assert k and 8 <= k[0]["registers"] <= 255 and k[0]["spill_stores"] == 0 and k[0]["smem_bytes"] > 0
    r2 = CR.compile_and_run(folder, str(src), build_only=True, work_dir=str(tmp_path / "b"))
    assert r2.compile_success and "[build cache hit]" in r2.compile_output and r2.ptxas == r1.ptxas
    src.write_text(src.read_text() + "\n// changed\n")
    r3 = CR.compile_and_run(folder, str(src), build_only=True, work_dir=str(tmp_path / "b"))
    assert r3.compile_success and "[build cache hit]" not in r3.compile_output
    ok, _, log, _ = CR.compile_source(str(src), str(tmp_path / "dbg"), debug=True)
    assert ok and "[build cache hit]" not in log


def test_ptxas_report_parser():
    log = ("ptxas info    : Compiling entry function '_Z1kPf' for 'sm_100a'\n"
           "ptxas info    : Function properties for _Z1kPf\n"
           "    16 bytes stack frame, 8 bytes spill stores, 12 bytes spill loads\n"
           "ptxas info    : Used 40 registers, used 1 barriers, 4096 bytes smem\n"
           "ptxas info    : Compiling entry function '_Z1jv' for 'sm_100a'\n"
           "    0 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads\n"
           "ptxas info    : Used 12 registers, used 0 barriers\n")
    assert CR.ptxas_report(log) == [
        {"kernel": "_Z1kPf", "registers": 40, "spill_stores": 8, "spill_loads": 12, "smem_bytes": 4096},
        {"kernel": "_Z1jv", "registers": 12, "spill_stores": 0, "spill_loads": 0, "smem_bytes": 0}]
