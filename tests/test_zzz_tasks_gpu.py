"""The shipped single-GPU tasks: every reference builds with nvcc for sm_100a, runs, and passes its
own check on the device; the unfilled skeleton does not pass."""
import os

import pytest

from commbench_b200.harness import compile_run as CR

pytestmark = pytest.mark.gpu

TASKS = os.path.join(os.path.dirname(CR.__file__), "tasks")
GPU1 = sorted((d for d in os.listdir(TASKS)
               if os.path.exists(os.path.join(TASKS, d, "task.json"))
               and CR.load_task(os.path.join(TASKS, d))["needs_gpu"]
               and CR.load_task(os.path.join(TASKS, d))["world"] == 1),
              key=lambda d: (CR.load_task(os.path.join(TASKS, d)).get("added", 0), d))   # oldest tasks first


@pytest.mark.timeout(600)
@pytest.mark.parametrize("task", GPU1)
def test_gpu_task_reference_passes_and_skeleton_does_not(task, tmp_path):
    folder = os.path.join(TASKS, task)
    r = CR.compile_and_run(folder, CR.find_ref_file(folder), work_dir=str(tmp_path))
    assert CR.analyze_result(r) == (True, "program reported PASS"), r.output[-2000:]
    rows = (r.result_json or {}).get("metrics")
    assert rows and all(CR.load_task(folder)["primary_metric"] in row for row in rows)
    skel = CR.compile_and_run(folder, CR.find_empty_file(folder), work_dir=str(tmp_path))
    assert skel.compile_success and not CR.analyze_result(skel)[0]
