"""The op registry: every reference example is mapped, every named API exists, every named task
is shipped, and the migration table has one row per example."""
import importlib
import os
import re

from commbench_b200.harness import compile_run as CR
from commbench_b200.harness import registry as R

TASKS = os.path.join(os.path.dirname(CR.__file__), "tasks")
# The reference's data set: example001 .. example102 without 036, 041, 071, plus 105 and 109.
EXPECTED = {f"example{n:03d}" for n in list(range(1, 103)) + [105, 109]} - {"example036", "example041", "example071"}


def test_every_reference_example_is_registered_once_per_row():
    covered = R.examples_covered()
    assert len(EXPECTED) == 101 and covered == EXPECTED, (sorted(EXPECTED - covered), sorted(covered - EXPECTED))
    rows = [l for l in R.migration_table().splitlines()[2:]]
    names = [l.split("|")[1].strip() for l in rows]
    assert set(names) == EXPECTED and len(names) >= 101
    assert all(l.count("|") == 5 for l in rows)


def test_info_only_ops_and_unknown_ops():
    assert R.entry("nanosleep") == "info_only" and R.entry("gpu_attributes") == "info_only"
    assert R.entry("all_reduce") == {"primary": "time_ms", "direction": "lower"}
    assert R.entry("p2p_copy")["direction"] == "higher" and R.entry("no_such_op") is None
    assert set(R.API) == set(R.OPS)


def _resolve(dotted: str) -> bool:
    parts = dotted.split(".")
    for cut in range(len(parts), 0, -1):
        try:
            obj = importlib.import_module("commbench_b200." + ".".join(parts[:cut]))
        except ImportError:
            continue
        for attr in parts[cut:]:
            if not hasattr(obj, attr):
                return False
            obj = getattr(obj, attr)
        return True
    return False


def test_every_named_api_and_task_exists():
    pat = re.compile(r"\b((?:ops|parallel|harness)\.[A-Za-z_][\w]*(?:\.[A-Za-z_]\w*)*)")
    texts = [a for a, _ in R.API.values()] + list(R.EXAMPLE_API.values())
    missing = []
    for text in texts:
        # "a.b.c / d" and "a.b.c, d" name siblings of the first object in the same module
        for m in pat.finditer(text):
            if not _resolve(m.group(1)):
                missing.append(m.group(1))
        for first, sib in re.findall(r"((?:ops|parallel)\.\w+)\.\w+(?:\s*[,/]\s*(\w+))+", text):
            if sib and not _resolve(f"{first}.{sib}"):
                missing.append(f"{first}.{sib}")
    assert not missing, missing
    shipped = set(os.listdir(TASKS))
    named = set(R.EXAMPLE_TASK.values())
    for _, t in R.API.values():
        named |= {x.strip() for x in (t or "").split(",") if x.strip()}
    assert named <= shipped, sorted(named - shipped)
