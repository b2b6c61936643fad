"""``python -m commbench_b200 <command> [args...]``: one front door to the command-line tools.

    run         the measurement suites (launch under torchrun for more than one GPU)
    profile     one small self-contained launch sequence per hot kernel
    task        build / run / compare one source file of a task
    eval        generate -> build -> run -> compare -> repair for one task
    leaderboard all tasks for one model, and the model table
    skeleton    derive a task's skeleton from its marked reference solution
    examples    where each example of the reference suite lives in this package
    platform    what this machine has (GPUs, toolchain, fabric, NICs)
    build       compile the native library in-tree
"""
from __future__ import annotations

import importlib
import sys

COMMANDS = {
    "run": "commbench_b200.harness.run",
    "profile": "commbench_b200.harness.profile_case",
    "task": "commbench_b200.harness.task_runner",
    "eval": "commbench_b200.harness.eval_driver",
    "leaderboard": "commbench_b200.harness.leaderboard",
    "skeleton": "commbench_b200.harness.make_skeleton",
    "examples": "commbench_b200.harness.registry",
    "platform": "commbench_b200.harness.platform_detect",
    "build": "commbench_b200._build",
}


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help", "help"):
        print(__doc__.strip())
        return 0
    cmd, rest = argv[0], argv[1:]
    if cmd not in COMMANDS:
        print(f"unknown command {cmd!r}; one of: {', '.join(COMMANDS)}", file=sys.stderr)
        return 2
    mod = importlib.import_module(COMMANDS[cmd])
    if cmd == "examples":
        print(mod.migration_table(), end="")
        return 0
    if cmd == "build":
        print(mod.build(force="--force" in rest, verbose="--verbose" in rest,
                        ptxas_verbose="--ptxas-verbose" in rest))
        return 0
    if not hasattr(mod, "main"):
        print(f"{COMMANDS[cmd]} has no command-line entry", file=sys.stderr)
        return 2
    try:
        rc = mod.main(rest)
    except TypeError:                  # an entry point that reads sys.argv itself
        sys.argv = [COMMANDS[cmd]] + rest
        rc = mod.main()
    return int(rc or 0)


if __name__ == "__main__":
    sys.exit(main())
