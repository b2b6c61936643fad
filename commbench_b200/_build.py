"""In-tree build of the native library.

Every ``.cu`` / ``.cc`` under ``csrc/`` is compiled for sm_100a and linked into
``commbench_b200/lib/libcommbench_b200.so`` (C ABI, loaded with ctypes).  Objects are cached
by a hash of the source, the headers it can see and the flags, the same idea as
the reference's mtime build cache
(datasets/example060_thunderkitten_all_reduce_hard/nv/build_and_run.py:227-242).

The flags mirror the reference's ThunderKittens builds
(``-gencode arch=compute_100a,code=sm_100a -std=c++20 -O3 -lineinfo
-Xptxas=--warn-on-spills``: same file, lines 189-202).
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import json
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
OBJDIR = PKG.parent / "build" / "obj"
LIBNAME = "libcommbench_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++20", "-O3", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xptxas=--warn-on-spills",
    "--expt-relaxed-constexpr",
    "-cudart", "static",
]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def sources() -> list[Path]:
    return sorted(list(CSRC.rglob("*.cu")) + list(CSRC.rglob("*.cc")))


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _key(src: Path, hdr: str, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    h.update(hdr.encode())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:24]


def _compile(nvcc: str, src: Path, obj: Path, flags: list[str], verbose: bool) -> tuple[Path, str]:
    cmd = [nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if src.suffix == ".cc" and src.name.startswith("transport_"):
        # Host-only C++ (containers of local types trip the CUDA front end): nvcc hands the file
        # to the host compiler, with the toolkit's include paths.
        host_flags = [f for f in flags if not f.startswith("-Xptxas") and f != "--expt-relaxed-constexpr"]
        cmd = [nvcc, *host_flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    elif src.suffix == ".cc":
        cmd = [nvcc, *flags, "-x", "cu", "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    log = (r.stdout or "") + (r.stderr or "")
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{' '.join(cmd)}\n{log}")
    if verbose and log.strip():
        print(log, file=sys.stderr)
    return obj, log


def build(force: bool = False, verbose: bool = False, ptxas_verbose: bool = False,
          jobs: int | None = None) -> Path:
    """Compiles what changed and links the shared object; returns its path."""
    nvcc = nvcc_path()
    flags = list(NVCC_FLAGS)
    if ptxas_verbose:
        flags.append("-Xptxas=-v")
    OBJDIR.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    hdr = _headers_digest()
    srcs = sources()
    manifest_path = OBJDIR / "manifest.json"
    try:
        manifest = json.loads(manifest_path.read_text())
    except Exception:
        manifest = {}
    todo: list[tuple[Path, Path, str]] = []
    objs: list[Path] = []
    for s in srcs:
        rel = s.relative_to(CSRC).as_posix().replace("/", "__")
        obj = OBJDIR / (rel + ".o")
        key = _key(s, hdr, flags)
        objs.append(obj)
        if force or not obj.exists() or manifest.get(rel) != key:
            todo.append((s, obj, key))
    logs = {}
    if todo:
        jobs = jobs or min(len(todo), os.cpu_count() or 4)
        with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
            futs = {ex.submit(_compile, nvcc, s, o, flags, verbose): (s, o, k) for s, o, k in todo}
            for f in cf.as_completed(futs):
                s, o, k = futs[f]
                _, log = f.result()
                logs[s.name] = log
                manifest[s.relative_to(CSRC).as_posix().replace("/", "__")] = k
        manifest_path.write_text(json.dumps(manifest, indent=1))
    lib = LIBDIR / LIBNAME
    if todo or not lib.exists():
        cmd = [nvcc, "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", str(lib), *map(str, objs), "-lrt", "-lpthread", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{' '.join(cmd)}\n{r.stdout}{r.stderr}")
    if ptxas_verbose:
        (OBJDIR / "ptxas.log").write_text("\n".join(f"== {k}\n{v}" for k, v in logs.items()))
    return lib


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-verbose", action="store_true",
                    help="pass -Xptxas=-v and keep the register/spill report in build/obj/ptxas.log")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose, ptxas_verbose=a.ptxas_verbose))
