"""ctypes binding of libstrix_b200.so, generated from include/strix_b200.h.

The prototypes are read from the header at import time so the Python side can
never drift from the C-ABI. There is no fallback: if the shared library is
missing or lacks a declared symbol, importing fails with the build command.
"""

from __future__ import annotations

import ctypes
import os
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
HEADER = PKG.parent / "include" / "strix_b200.h"
LIB_PATH = PKG / "libstrix_b200.so"

STRIX_OK = 0

_CTYPES = {
    "void": None,
    "int": ctypes.c_int,
    "int32_t": ctypes.c_int32,
    "int64_t": ctypes.c_int64,
    "float": ctypes.c_float,
    "double": ctypes.c_double,
    "strix_stream_t": ctypes.c_void_p,
}

_DECL = re.compile(
    r"^\s*((?:const\s+)?[A-Za-z_][A-Za-z0-9_]*\s*\**)\s*(strix_[a-z0-9_]+)\s*\(([^;{}]*)\)\s*;",
    re.M | re.S,
)


def _ctype(text: str):
    t = text.replace("const", " ").strip()
    if "*" in t:
        base = t.replace("*", "").strip()
        return ctypes.c_char_p if base == "char" else ctypes.c_void_p
    return _CTYPES[t]


def parse_header(path: Path = HEADER) -> dict[str, tuple]:
    """name -> (restype, [argtypes], [argnames]) for every function the header declares."""
    src = re.sub(r"/\*.*?\*/", "", path.read_text(), flags=re.S)
    src = re.sub(r"//[^\n]*", "", src)
    src = re.sub(r"^\s*#.*$", "", src, flags=re.M)
    protos = {}
    for ret, name, args in _DECL.findall(src):
        args = " ".join(args.split())
        argtypes, argnames = [], []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                m = re.match(r"^(.*?)([A-Za-z_][A-Za-z0-9_]*)$", a)
                argtypes.append(_ctype(m.group(1)))
                argnames.append(m.group(2))
        protos[name] = (_ctype(ret), argtypes, argnames)
    return protos


class StrixError(RuntimeError):
    """A C-ABI call rejected its arguments or a CUDA call failed."""


_lib = None
_protos: dict[str, tuple] = {}


def load() -> ctypes.CDLL:
    """Loads the shared library once and types every declared entry point."""
    global _lib, _protos
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python libstrix_b200/build.py` "
            "(needs nvcc; there is no CPU or PyTorch fallback)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    _protos = parse_header()
    for name, (ret, argtypes, _) in _protos.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise ImportError(
                f"{LIB_PATH} does not export {name}; rebuild it with "
                "`python libstrix_b200/build.py`") from e
        fn.restype = ret
        fn.argtypes = argtypes
    _lib = lib
    return lib


def prototypes() -> dict[str, tuple]:
    load()
    return dict(_protos)


def call(name: str, *args) -> None:
    """Calls a status-returning entry point; raises StrixError with the library's message."""
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != STRIX_OK:
        msg = lib.strix_last_error().decode("utf-8", "replace")
        raise StrixError(msg or f"{name} failed with status {rc}")


def umma_status() -> int:
    """The health word of the tcgen05 kernels on the current device (synchronises it):
    0 while every launch met its bounded waits, 1 after one gave up."""
    flag = ctypes.c_int32(-1)
    call("strix_umma_status", ctypes.byref(flag))
    return flag.value


# STRIX_CHECK_STATUS=1: every op that runs a tcgen05 kernel synchronises afterwards
# and raises if a bounded wait gave up (its output is then incomplete). Off by
# default - the check costs a device synchronisation per call; a serving loop polls
# umma_status() at a point where it synchronises anyway.
CHECK_STATUS = os.environ.get("STRIX_CHECK_STATUS", "") not in ("", "0")


def after_tcgen05(op: str) -> None:
    if CHECK_STATUS and umma_status() != 0:
        raise StrixError(f"{op}: a bounded wait of a tcgen05 kernel gave up; the output is incomplete")
