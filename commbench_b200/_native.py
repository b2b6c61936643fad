"""ctypes binding of ``lib/libcommbench_b200.so`` (C ABI).

The library is built in-tree by :mod:`commbench_b200._build`; importing this module never
compiles anything unless ``CB200_AUTOBUILD=1``.  On a machine with a GPU a missing
library is an error (no silent PyTorch fallback): ops that need it raise.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

MAX_RANKS = 8
PAD_CHANNELS = 1024
PAD_NVLS_BASE = PAD_CHANNELS * MAX_RANKS
PAD_ABORT = PAD_NVLS_BASE + PAD_CHANNELS
PAD_WORDS = PAD_ABORT + 64

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libcommbench_b200.so"
_lib = None


class NativeError(RuntimeError):
    pass


class CbComm(C.Structure):
    _fields_ = [
        ("rank", C.c_int32),
        ("world", C.c_int32),
        ("pad", C.c_void_p * MAX_RANKS),
        ("mc_pad", C.c_void_p),
        ("epoch", C.c_void_p),
        ("status", C.c_void_p),
        ("timeout_ns", C.c_uint64),
        ("jitter_ns", C.c_uint32),
        ("reserved", C.c_uint32),
    ]


class CollArgs(C.Structure):
    _fields_ = [
        ("comm", CbComm),
        ("sym", C.c_void_p * MAX_RANKS),
        ("mc", C.c_void_p),
        ("inp", C.c_void_p),
        ("out", C.c_void_p),
        ("nbytes", C.c_ulonglong),
        ("copy_in", C.c_int),
        ("copy_out", C.c_int),
        ("root", C.c_int),
        ("dtype", C.c_int),
        ("a2a_b", C.c_int),
        ("a2a_s_local", C.c_int),
        ("a2a_h", C.c_int),
        ("a2a_d", C.c_int),
        ("a2a_to_heads", C.c_int),
        ("unroll", C.c_int),
        ("variant", C.c_int),
    ]


# op codes of cb_coll_launch
OP_AR_ONESHOT, OP_AR_TWOSHOT, OP_AR_NVLS, OP_AG_PULL, OP_AG_PUSH, OP_RS, OP_A2A_FLAT, OP_A2A_4D, \
    OP_BCAST = range(9)
DT_BF16, DT_F16, DT_F32 = 0, 1, 2

STATUS_CODES = {
    0: "ok",
    1: "timeout waiting for a peer GPU's flag",
    2: "timeout on an mbarrier inside a CTA",
    3: "timeout waiting for another CTA's flag",
    4: "a peer aborted",
    5: "bad argument detected on the device",
    6: "timeout waiting for a host-written flag",
}


def decode_status(word: int) -> str:
    code, phase, detail = word >> 24, (word >> 16) & 0xFF, word & 0xFFFF
    return f"{STATUS_CODES.get(code, f'code {code}')} (phase {phase}, detail {detail})"


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def load():
    """Returns the loaded library, building it first only if CB200_AUTOBUILD=1."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        if os.environ.get("CB200_AUTOBUILD", "0") == "1":
            from . import _build

            _build.build()
        else:
            raise NativeError(
                f"{_LIB_PATH} is missing: run `python -m commbench_b200._build` "
                "(or __graft_entry__.build()) first")
    lib = C.CDLL(str(_LIB_PATH), mode=C.RTLD_GLOBAL)
    lib.cb_last_error.restype = C.c_char_p
    for name in ("cb_symm_round_size",):
        getattr(lib, name).restype = C.c_longlong
    if lib.cb_sizeof_coll_args() != C.sizeof(CollArgs):
        raise NativeError(
            f"CollArgs layout mismatch: C {lib.cb_sizeof_coll_args()} vs ctypes {C.sizeof(CollArgs)}")
    _lib = lib
    return lib


def last_error() -> str:
    lib = load()
    s = lib.cb_last_error()
    return s.decode() if s else ""


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what} failed (rc={rc}): {last_error()}")


def ptr(t) -> C.c_void_p:
    """Device pointer of a torch tensor (or None)."""
    return C.c_void_p(0 if t is None else t.data_ptr())


def stream_ptr(stream=None) -> C.c_void_p:
    import torch

    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)
