"""ctypes front end of the C restatement (oracle/w4a16_oracle.c).  TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force: bool = False) -> str:
    so = os.path.join(_HERE, "libglowq_oracle.so")
    src = os.path.join(_HERE, "w4a16_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B", "libglowq_oracle.so"])
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
        _LIB.glowq_oracle_max_threads.restype = ctypes.c_int
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def max_threads() -> int:
    return int(lib().glowq_oracle_max_threads())


def dequant(qweight, scales, qzeros, IC: int, group_size: int) -> np.ndarray:
    qweight, scales, qzeros = (np.ascontiguousarray(a) for a in (qweight, scales, qzeros))
    OC = qweight.shape[0]
    out = np.empty((OC, IC), dtype=np.float16)
    rc = lib().glowq_oracle_dequant(_p(qweight), _p(scales), _p(qzeros), _p(out), OC, IC, group_size,
                                    qweight.shape[1], qzeros.shape[1], scales.shape[1])
    if rc:
        raise RuntimeError(f"glowq_oracle_dequant failed: {rc}")
    return out


def corrected_forward(x, qweight, scales, qzeros, group_size, bias=None, R=None, L=None, alpha=1.0,
                      r_io=None, r_mode=None, num_threads=0) -> np.ndarray:
    """fp32 [M, OC].  r_mode None: 1 when R and L are given, else 0."""
    x, qweight, scales, qzeros = (np.ascontiguousarray(a) for a in (x, qweight, scales, qzeros))
    M, IC = x.shape
    OC = qweight.shape[0]
    if r_mode is None:
        r_mode = 1 if (R is not None and L is not None) else 0
    rank = 0 if L is None else L.shape[1]
    if r_mode and r_io is None:
        r_io = np.zeros((M, rank), dtype=np.float32)
    R = None if R is None else np.ascontiguousarray(R)
    L = None if L is None else np.ascontiguousarray(L)
    bias = None if bias is None else np.ascontiguousarray(bias)
    y = np.empty((M, OC), dtype=np.float32)
    rc = lib().glowq_oracle_corrected_forward(
        _p(x), _p(qweight), _p(scales), _p(qzeros), _p(bias), _p(R), _p(L), _p(r_io), int(r_mode),
        ctypes.c_float(alpha), _p(y), M, IC, OC, rank, group_size, qweight.shape[1], qzeros.shape[1],
        scales.shape[1], int(num_threads))
    if rc:
        raise RuntimeError(f"glowq_oracle_corrected_forward failed: {rc}")
    return y
