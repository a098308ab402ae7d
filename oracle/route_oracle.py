"""ctypes front end of ``route_oracle.c`` (CPU oracle, test infrastructure only)."""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libroute_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ``route_oracle.c`` with gcc into ``oracle/_build``."""
    src = os.path.join(_HERE, "route_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _SO


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
    return _lib


def _p(a, t):
    return a.ctypes.data_as(ctypes.POINTER(t))


def topk_mask(logits: np.ndarray, keep: int) -> np.ndarray:
    l = np.ascontiguousarray(logits, dtype=np.float32)
    ng = l.shape[-1]
    rows = l.size // ng
    out = np.zeros(l.shape, dtype=np.uint8)
    rc = _load().oracle_topk_mask(_p(l, ctypes.c_float), ctypes.c_int64(rows), ng, keep,
                                  _p(out, ctypes.c_uint8))
    if rc:
        raise ValueError("keep out of range")
    return out.astype(bool)


def route_compact(mask2d: np.ndarray):
    m8 = np.ascontiguousarray(mask2d, dtype=np.uint8)
    M, NG = m8.shape
    smask = np.zeros((M, NG), dtype=np.uint8)
    sidx = np.zeros((M, NG), dtype=np.int64)
    counts = np.zeros((NG,), dtype=np.int32)
    _load().oracle_route_compact(_p(m8, ctypes.c_uint8), ctypes.c_int64(M), NG,
                                 _p(smask, ctypes.c_uint8), _p(sidx, ctypes.c_int64),
                                 _p(counts, ctypes.c_int32))
    return smask.astype(bool), sidx, counts


def row_bits(mask2d: np.ndarray, window: int = 128):
    m8 = np.ascontiguousarray(mask2d, dtype=np.uint8)
    M, NG = m8.shape
    words = (NG + 31) // 32
    nwin = (M + window - 1) // window
    rb = np.zeros((M, words), dtype=np.uint32)
    wb = np.zeros((nwin, words), dtype=np.uint32)
    _load().oracle_row_bits(_p(m8, ctypes.c_uint8), ctypes.c_int64(M), NG, window,
                            _p(rb, ctypes.c_uint32), _p(wb, ctypes.c_uint32))
    return rb, wb
