"""Loader of the sm_100a C-ABI library and torch-tensor front ends of its entry points.

Counterpart of GlowQ's ``cuda_w4a16/kernels.py`` (``load_w4a16_extension``, src/cuda_w4a16/kernels.py:16-59)
and of the three names its pybind module exports (src/cuda_w4a16/csrc/pybind.cpp:19-34).  There is no JIT
fallback and no other backend: if the library is missing or the device is not sm_100, calls raise."""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_NAME = "libglowq_w4a16.so"

GLOWQ_OK = 0
ERR_DEVICE_TIMEOUT = 7
OUT_F16, OUT_F32 = 0, 1
R_NONE, R_COMPUTE, R_LOAD = 0, 1, 2
KERNEL_AUTO, KERNEL_GEMV, KERNEL_GEMM = 0, 1, 2
MAX_MEMBERS = 4
ABI_VERSION = 2


class Member(ctypes.Structure):
    _fields_ = [("qweight", ctypes.c_void_p), ("scales", ctypes.c_void_p), ("qzeros", ctypes.c_void_p),
                ("bias", ctypes.c_void_p), ("L", ctypes.c_void_p), ("out", ctypes.c_void_p),
                ("OC", ctypes.c_int32), ("weight_stride_i32", ctypes.c_int32), ("zero_stride_i32", ctypes.c_int32),
                ("scale_stride", ctypes.c_int32), ("L_stride", ctypes.c_int32), ("out_stride", ctypes.c_int32),
                ("alpha", ctypes.c_float), ("reserved", ctypes.c_int32)]


class Group(ctypes.Structure):
    _fields_ = [("x", ctypes.c_void_p), ("R", ctypes.c_void_p), ("r_buf", ctypes.c_void_p),
                ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t), ("stream", ctypes.c_void_p),
                ("M", ctypes.c_int32), ("IC", ctypes.c_int32), ("x_stride", ctypes.c_int32),
                ("R_stride", ctypes.c_int32), ("rank", ctypes.c_int32), ("group_size", ctypes.c_int32),
                ("r_mode", ctypes.c_int32), ("out_dtype", ctypes.c_int32), ("kernel", ctypes.c_int32),
                ("n_members", ctypes.c_int32), ("split_k", ctypes.c_int32), ("reserved", ctypes.c_int32),
                ("next", ctypes.c_void_p),     # address of the Group that follows on the stream, or None
                ("push", ctypes.c_void_p),     # address of a Peers struct: push the result to every rank (row-split TP)
                ("push_site", ctypes.c_int32), ("reserved2", ctypes.c_int32),
                ("norm_weight", ctypes.c_void_p), ("residual", ctypes.c_void_p), ("hidden_out", ctypes.c_void_p),
                ("norm_eps", ctypes.c_float), ("reserved3", ctypes.c_int32),
                ("members", Member * MAX_MEMBERS)]


MAX_RANKS = 8


class Peers(ctypes.Structure):
    _fields_ = [("buf", ctypes.c_void_p * MAX_RANKS), ("flag", ctypes.c_void_p * MAX_RANKS), ("epoch", ctypes.c_void_p),
                ("status", ctypes.c_void_p), ("world", ctypes.c_int32), ("rank", ctypes.c_int32),
                ("sites", ctypes.c_int32), ("max_n", ctypes.c_int32), ("ll_buf", ctypes.c_void_p * MAX_RANKS)]


EXPORTS = ("glowq_w4a16_version", "glowq_w4a16_strerror", "glowq_w4a16_last_cuda_error", "glowq_w4a16_dequant",
           "glowq_w4a16_gemv_forward", "glowq_w4a16_gemm_forward", "glowq_w4a16_group_forward",
           "glowq_w4a16_group_forward_many", "glowq_w4a16_group_forward_host", "glowq_w4a16_workspace_bytes",
           "glowq_w4a16_read_status", "glowq_w4a16_gemv_forward_static", "glowq_w4a16_allreduce_f16",
           "glowq_w4a16_allreduce_finish_f16")


def library_path() -> str:
    env = os.environ.get("GLOWQ_W4A16_LIB")
    cands = ([env] if env else []) + [os.path.join(_HERE, _LIB_NAME), os.path.join(os.path.dirname(_HERE), _LIB_NAME)]
    for c in cands:
        if c and os.path.exists(c):
            return c
    raise RuntimeError(
        f"{_LIB_NAME} not found (looked in {cands}). Build it with `python -m glowq_b200.build`; "
        "this package has no JIT, Triton or CPU fallback.")


class _Ext:
    """What ``load_w4a16_extension()`` returns: the reference's three callables on torch tensors, plus ``lib``
    (the raw ctypes library) for the fused entry points."""

    def __init__(self, lib: ctypes.CDLL):
        self.lib = lib
        vp, i32, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
        lib.glowq_w4a16_version.restype = i32
        lib.glowq_w4a16_strerror.restype = ctypes.c_char_p
        lib.glowq_w4a16_strerror.argtypes = [i32]
        lib.glowq_w4a16_last_cuda_error.restype = i32
        lib.glowq_w4a16_dequant.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp]
        lib.glowq_w4a16_gemv_forward.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp, sz, vp]
        lib.glowq_w4a16_gemm_forward.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp, sz, vp]
        lib.glowq_w4a16_group_forward.argtypes = [ctypes.POINTER(Group)]
        lib.glowq_w4a16_group_forward_many.argtypes = [ctypes.POINTER(Group), i32]
        lib.glowq_w4a16_group_forward_host.argtypes = [ctypes.POINTER(Group), vp, ctypes.POINTER(vp)]
        lib.glowq_w4a16_workspace_bytes.restype = sz
        lib.glowq_w4a16_workspace_bytes.argtypes = [i32, i32, i32, i32, i32]
        lib.glowq_w4a16_read_status.argtypes = [vp, vp]
        lib.glowq_w4a16_gemv_forward_static.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp]
        lib.glowq_w4a16_allreduce_f16.argtypes = [ctypes.POINTER(Peers), vp, i32, i32, vp]
        lib.glowq_w4a16_allreduce_finish_f16.argtypes = [ctypes.POINTER(Peers), vp, i32, i32, vp]
        if lib.glowq_w4a16_version() != ABI_VERSION:
            raise RuntimeError("libglowq_w4a16.so ABI version mismatch; rebuild with `python -m glowq_b200.build`")
        self._ws = {}

    # ------------------------------------------------------------------ helpers
    def check(self, rc: int, what: str = "glowq_w4a16") -> None:
        if rc != GLOWQ_OK:
            msg = self.lib.glowq_w4a16_strerror(rc).decode()
            if rc == 6:
                msg += f" [cudaError {self.lib.glowq_w4a16_last_cuda_error()}]"
            raise RuntimeError(f"{what}: {msg} (status {rc})")

    def workspace_bytes(self, M: int, IC: int, OC_total: int, rank: int, n_members: int) -> int:
        return int(self.lib.glowq_w4a16_workspace_bytes(M, IC, OC_total, rank, n_members))

    def new_workspace(self, nbytes: int, device) -> torch.Tensor:
        """Zero-initialised workspace (the kernels re-arm their counters themselves after every launch)."""
        return torch.zeros(max(int(nbytes), 256), dtype=torch.uint8, device=device)

    def _scratch(self, device, nbytes: int) -> torch.Tensor:
        key = (device.type, device.index)
        ws = self._ws.get(key)
        if ws is None or ws.numel() < nbytes:
            ws = self.new_workspace(nbytes, device)
            self._ws[key] = ws
        return ws

    @staticmethod
    def _check_inputs(x, qweight, scales, qzeros, group_size):
        for t, name in ((x, "inputs"), (qweight, "qweight"), (scales, "scales"), (qzeros, "qzeros")):
            if not t.is_cuda:
                raise RuntimeError(f"{name} must be CUDA")
        if x.dtype != torch.float16:
            raise RuntimeError("inputs must be fp16")
        if qweight.dtype != torch.int32:
            raise RuntimeError("qweight must be int32 (8x int4 packed)")
        if scales.dtype != torch.float16:
            raise RuntimeError("scales must be fp16")
        if qzeros.dtype != torch.int32:
            raise RuntimeError("qzeros must be int32 (8x int4 packed)")
        if x.dim() != 2 or qweight.dim() != 2 or scales.dim() != 2 or qzeros.dim() != 2:
            raise RuntimeError("inputs must be [M, IC]; qweight [OC, packed]; scales [OC, groups]; qzeros [OC, groups_packed]")
        if group_size <= 0 or group_size % 8 != 0:
            raise RuntimeError("group_size must be > 0 and a multiple of 8")
        if scales.size(0) != qweight.size(0) or qzeros.size(0) != qweight.size(0):
            raise RuntimeError("scales / qzeros OC mismatch")

    def _plain(self, fn_name, x, qweight, scales, qzeros, group_size, extra=()):
        self._check_inputs(x, qweight, scales, qzeros, group_size)
        x, qweight, scales, qzeros = (t.contiguous() for t in (x, qweight, scales, qzeros))
        M, IC = x.shape
        OC = qweight.size(0)
        out = torch.empty((M, OC), dtype=torch.float16, device=x.device)
        if M == 0:
            return out
        with torch.cuda.device(x.device):
            ws = self._scratch(x.device, self.workspace_bytes(M, IC, OC, 0, 1))
            stream = torch.cuda.current_stream(x.device).cuda_stream
            fn = getattr(self.lib, fn_name)
            rc = fn(x.data_ptr(), qweight.data_ptr(), scales.data_ptr(), qzeros.data_ptr(), out.data_ptr(), M, IC, OC,
                    int(group_size), *extra, qweight.size(1), qzeros.size(1), scales.size(1), ws.data_ptr(), ws.numel(),
                    stream)
        self.check(rc, fn_name)
        return out

    # ------------------------------------------------------------------ the reference's three exports
    def w4a16_gemv_forward_cuda(self, x, qweight, scales, qzeros, group_size: int) -> torch.Tensor:
        """[M, OC] fp16 = x . dequant(Q)^T (csrc/gemv_w4a16.cu:146-214)."""
        return self._plain("glowq_w4a16_gemv_forward", x, qweight, scales, qzeros, group_size)

    gemv_w4a16_asym = w4a16_gemv_forward_cuda

    def w4a16_gemm_forward_cuda(self, x, qweight, scales, qzeros, group_size: int, split_k_iters: int = 1) -> torch.Tensor:
        """Same product through the tensor-core kernel (csrc/gemm_w4a16.cu:76-135); split_k_iters is ignored."""
        return self._plain("glowq_w4a16_gemm_forward", x, qweight, scales, qzeros, group_size, (int(split_k_iters),))

    def dequant(self, qweight, scales, qzeros, in_features: int, group_size: int) -> torch.Tensor:
        """[OC, in_features] fp16 dequantised weight, bit-exact with ``_dequant_chunk`` (linear.py:248-253)."""
        qweight, scales, qzeros = (t.contiguous() for t in (qweight, scales, qzeros))
        out = torch.empty((qweight.size(0), in_features), dtype=torch.float16, device=qweight.device)
        with torch.cuda.device(qweight.device):
            rc = self.lib.glowq_w4a16_dequant(qweight.data_ptr(), scales.data_ptr(), qzeros.data_ptr(), out.data_ptr(),
                                              qweight.size(0), in_features, int(group_size), qweight.size(1),
                                              qzeros.size(1), scales.size(1),
                                              torch.cuda.current_stream(qweight.device).cuda_stream)
        self.check(rc, "glowq_w4a16_dequant")
        return out


_ext: Optional[_Ext] = None


def load_w4a16_extension(verbose: Optional[bool] = None) -> _Ext:
    """Load (once) and return the kernel library front end (src/cuda_w4a16/kernels.py:16-59)."""
    global _ext
    if _ext is None:
        path = library_path()
        try:
            lib = ctypes.CDLL(path)
        except OSError as exc:
            raise RuntimeError(f"failed to load {path}: {exc}. Rebuild with `python -m glowq_b200.build`.") from exc
        missing = [n for n in EXPORTS if not hasattr(lib, n)]
        if missing:
            raise RuntimeError(f"{path} lacks symbols {missing}")
        _ext = _Ext(lib)
        if verbose:
            print(f"[glowq_b200] loaded {path}")
    return _ext


__all__ = ["load_w4a16_extension"]
