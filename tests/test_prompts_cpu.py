"""The prompt variants beyond completion / fix: detailed completion, optimisation prompts."""
import os

from commbench_b200.harness import compile_run as CR
from commbench_b200.harness.llm import prompt as P

TASKS = os.path.join(os.path.dirname(CR.__file__), "tasks")


def test_detailed_completion_prompt_names_machine_and_hints():
    skel = CR.find_empty_file(os.path.join(TASKS, "mbarrier_producer_consumer"))
    plain = P.generate_completion_prompt(skel, "Fill it in.")
    det = P.generate_completion_prompt_detailed(skel, "Fill it in.", hints=["arrive has release semantics"])
    assert det.startswith(plain.rstrip("\n")) and "Machine:" in det and "sm_100a" in det
    assert "- arrive has release semantics" in det and "NVLink 5" in det
    own = P.generate_completion_prompt_detailed(skel, hardware={"gpu": "test part"})
    assert "- gpu: test part" in own and "Hints:" not in own and "NVLink" not in own.split("Machine:")[1]


def test_optimisation_prompts_carry_program_rules_and_numbers():
    ref = CR.find_ref_file(os.path.join(TASKS, "gloo_allreduce"))
    p = P.generate_optimization_prompt(ref, goal="higher bandwidth")
    assert "higher bandwidth" in p and "```python" in p and "dist.all_reduce" in p
    assert "Reply with the complete source file" in p
    q = P.generate_performance_optimization_prompt(ref, {"latency_avg": 812.5, "throughput_avg": 5.1},
                                                   roofline={"fraction_of_link": 0.04})
    assert '"latency_avg": 812.5' in q and '"fraction_of_link": 0.04' in q and "bottleneck" in q
    cu = CR.find_ref_file(os.path.join(TASKS, "d2d_copy_kernel"))
    r = P.generate_performance_optimization_prompt(cu, {"throughput_avg": 3000.0})
    assert "```cuda" in r and "Against the machine's limits" not in r and "bounded" in r
    big = P.generate_performance_optimization_prompt(ref, {"rows": ["x" * 100] * 100})
    assert "characters omitted" in big                      # long metric dumps are capped
