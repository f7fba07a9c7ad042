"""The C part of the CPU oracle (``e8_oracle.c``), built with gcc and bound with ctypes.

TEST INFRASTRUCTURE: a second, independent restatement of the decode (the first is numpy,
``oracle/e8.py``), fast enough to decode whole experts in tests and in the benchmark's CPU
baseline.  Only tests, ``__graft_entry__`` and ``bench.py`` may use it.
"""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIBRARY = HERE / "libe8oracle.so"
_lib = None


def build(force: bool = False) -> Path:
    source = HERE / "e8_oracle.c"
    if force or not LIBRARY.exists() or LIBRARY.stat().st_mtime < source.stat().st_mtime:
        subprocess.run(["gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-o", str(LIBRARY), str(source)], check=True)
    return LIBRARY


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(str(build()))
        p, i64 = ctypes.c_void_p, ctypes.c_int64
        lib.e8p_decode.argtypes, lib.e8p_decode.restype = [p, i64, p, p], None
        lib.e8_1bit_decode.argtypes, lib.e8_1bit_decode.restype = [p, i64, p, p], None
        lib.vq_qmv.argtypes, lib.vq_qmv.restype = [p, p, i64, i64, i64, p, p, p], None
        _lib = lib
    return _lib


def _ptr(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def decode_e8p(codes, abs_table) -> np.ndarray:
    """uint16 codes of any shape -> float32 ``codes.shape + (8,)``."""
    c = np.ascontiguousarray(codes, dtype=np.uint16)
    t = np.ascontiguousarray(abs_table, dtype=np.uint32)
    out = np.empty(c.shape + (8,), dtype=np.float32)
    load().e8p_decode(_ptr(c), c.size, _ptr(t), _ptr(out))
    return out


def decode_e8_1bit(codes, table) -> np.ndarray:
    c = np.ascontiguousarray(codes, dtype=np.uint8)
    t = np.ascontiguousarray(table, dtype=np.uint32)
    out = np.empty(c.shape + (8,), dtype=np.float32)
    load().e8_1bit_decode(_ptr(c), c.size, _ptr(t), _ptr(out))
    return out


def vq_qmv(x, codes, scales, abs_table) -> np.ndarray:
    """``decode_weight_matrix(codes, scales) @ x`` for one matrix: codes ``[out, in/8]`` uint16,
    scales ``[out, groups]``, x ``[in]`` -> float64 ``[out]``."""
    c = np.ascontiguousarray(codes, dtype=np.uint16)
    s = np.ascontiguousarray(scales, dtype=np.float32)
    v = np.ascontiguousarray(x, dtype=np.float32)
    t = np.ascontiguousarray(abs_table, dtype=np.uint32)
    out = np.empty(c.shape[0], dtype=np.float64)
    load().vq_qmv(_ptr(c), _ptr(s), c.shape[0], c.shape[1], s.shape[1], _ptr(v), _ptr(t), _ptr(out))
    return out
