"""Drop-in ``cuda_w4a16.linear``: RTN uint4 quantiser/packer, the replacement module ``CudaW4A16Linear``
(same constructor, buffers, attributes and ``from_float`` as src/cuda_w4a16/linear.py:91-276) and the
model-conversion pass ``convert_to_cuda_w4a16`` (linear.py:279-293), on top of the sm_100a C-ABI library.

Differences from the reference, all on the host side of the same interface:
* forward runs only on CUDA tensors of an sm_100 device; there is no pure-torch or CPU path;
* the kernel choice knobs W4A16_KERNEL_OUT_DTYPE / W4A16_GEMV_M_MAX / W4A16_FORCE_GEMM / W4A16_FORCE_GEMV are
  read once when the module is built (the reference re-reads the environment on every call, linear.py:172-177);
  W4A16_GEMV_M_MAX has no built-in default of 128 here: unset, the library switches kernels where it measured the
  cross-over (8 tokens);
  the dequant-cache / chunk / JIT knobs belong to fallbacks that do not exist here;
* output and scratch buffers are caller-side torch tensors; the library allocates nothing.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch
import torch.nn as nn

from . import kernels as K
from .kernels import load_w4a16_extension

_TRUE = {"1", "true", "yes", "y", "on"}


def _env_flag(*names: str) -> bool:
    for n in names:
        v = os.environ.get(n)
        if v is not None:
            return v.lower() in _TRUE
    return False


def _env_int(*names: str, default: int) -> int:
    for n in names:
        v = os.environ.get(n)
        if v:
            return int(v)
    return int(default)


def _get_kernel_out_dtype() -> torch.dtype:
    """W4A16_KERNEL_OUT_DTYPE (legacy MIXED_KERNEL_OUT_DTYPE), default fp32 (linear.py:29-39)."""
    v = os.environ.get("W4A16_KERNEL_OUT_DTYPE", os.environ.get("MIXED_KERNEL_OUT_DTYPE", "fp32")).lower()
    return torch.float16 if v in ("fp16", "float16", "half") else torch.float32


def _pack_int4_to_int32(u4: torch.Tensor) -> torch.Tensor:
    """[..., 8] uint8 codes -> [...] int32 with code j in bits [4j, 4j+4) (linear.py:42-46)."""
    if u4.dtype != torch.uint8 or u4.shape[-1] != 8:
        raise ValueError("expected uint8 codes with a trailing axis of 8")
    word = torch.zeros(u4.shape[:-1], dtype=torch.int32, device=u4.device)
    for j in range(8):
        word |= u4[..., j].to(torch.int32) << (4 * j)   # bit 31 wraps into the sign, as int32 arithmetic does
    return word


def _unpack_int4_i32(packed_i32: torch.Tensor, total_vals: int) -> torch.Tensor:
    """Row-wise inverse of the packer (linear.py:49-54)."""
    p = packed_i32.contiguous().to(torch.int32)
    cols = [((p >> (4 * j)) & 0xF).to(torch.uint8) for j in range(8)]
    return torch.stack(cols, dim=-1).reshape(p.size(0), -1)[:, :total_vals].contiguous()


def _quantize_per_group_w4(weight: torch.Tensor, group_size: int):
    """RTN asymmetric uint4 per (row, group) in the weight's own (fp16) arithmetic; returns
    (qweight_i32 [OC, ICp/8], qzeros_i32 [OC, ceil(G/8)], scales_f16 [OC, G], ICp) exactly as
    src/cuda_w4a16/linear.py:57-88 does: scale = (max-min)/15, zero = round(-min/scale) clamped to [0,15],
    code = round(w/scale + zero) clamped to [0,15]; columns padded with zeros to a whole group; unused
    zero-point nibbles hold 8."""
    if group_size % 8 != 0:
        raise ValueError("group_size must be multiple of 8 for int32 int4 packing")
    oc, ic = weight.shape
    rem = ic % group_size
    if rem:
        weight = torch.nn.functional.pad(weight, (0, group_size - rem))
        ic = weight.shape[1]
    n_groups = ic // group_size
    grouped = weight.reshape(oc, n_groups, group_size)
    lo = grouped.amin(dim=-1)
    hi = grouped.amax(dim=-1)
    scales = ((hi - lo) / 15.0).clamp(min=1e-8)
    zeros = (-lo / scales).round().clamp(0, 15)
    codes = (grouped / scales[..., None] + zeros[..., None]).round().clamp(0, 15).to(torch.uint8)
    qweight = _pack_int4_to_int32(codes.view(oc, n_groups, group_size // 8, 8)).reshape(oc, ic // 8)

    words = (n_groups + 7) // 8
    z8 = torch.nn.functional.pad(zeros.to(torch.uint8), (0, words * 8 - n_groups), value=8)
    qzeros = _pack_int4_to_int32(z8.view(oc, words, 8))
    return qweight.contiguous(), qzeros.contiguous(), scales.to(torch.float16).contiguous(), ic


class CudaW4A16Linear(nn.Module):
    """W4A16 linear on packed int4 weights (src/cuda_w4a16/linear.py:91-276)."""

    def __init__(self, in_features: int, out_features: int, group_size: int = 128, bias: bool = False):
        super().__init__()
        self.in_features = int(in_features)
        self.out_features = int(out_features)
        self.group_size = int(group_size)
        if self.group_size <= 0 or self.group_size % 8 != 0:
            raise ValueError("group_size must be > 0 and a multiple of 8 for GlowQ int32 int4 packing")
        groups = math.ceil(self.in_features / self.group_size)
        groups_packed = (groups + 7) // 8
        self.register_buffer("qweight_i32", torch.empty(self.out_features, (self.in_features + 7) // 8, dtype=torch.int32))
        self.register_buffer("qzeros_i32", torch.empty(self.out_features, max(1, groups_packed), dtype=torch.int32))
        self.register_buffer("scales_f16", torch.empty(self.out_features, groups, dtype=torch.float16))
        self.register_buffer("gid", torch.arange(self.in_features, dtype=torch.long) // self.group_size, persistent=False)
        self.groups = groups
        self.groups_packed = groups_packed
        self.bias = nn.Parameter(torch.empty(self.out_features, dtype=torch.float16)) if bias else None

        self._ext = None
        # -1: the knob is unset and the library's own switch-over applies
        self._gemv_threshold = _env_int("W4A16_GEMV_M_MAX", "CUDA_MIXED_GEMV_M_MAX", default=-1)
        self._force_gemm = _env_flag("W4A16_FORCE_GEMM", "CUDA_MIXED_FORCE_GEMM")
        self._force_gemv = _env_flag("W4A16_FORCE_GEMV", "CUDA_MIXED_FORCE_GEMV") or _env_flag("W4A16_USE_GEMV")
        self._out_dtype = _get_kernel_out_dtype()
        self._check_status = _env_flag("GLOWQ_CHECK_STATUS")
        self._ws: Optional[torch.Tensor] = None      # scratch for plain (uncorrected) calls
        self._ws_key = None

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"group_size={self.group_size}, bias={self.bias is not None}")

    # ------------------------------------------------------------------ plumbing
    def _get_ext(self):
        if self._ext is None:
            self._ext = load_w4a16_extension()
        return self._ext

    def kernel_choice(self, m: int) -> int:
        """Which kernel a call with ``m`` tokens asks for (linear.py:172-181): a FORCE knob wins; otherwise an
        explicitly set W4A16_GEMV_M_MAX sends ``m <= W4A16_GEMV_M_MAX`` to the weight-streaming kernel and anything
        larger to the tensor-core kernel; with the knob unset the library's own switch-over (8 tokens) applies."""
        if self._force_gemm:
            return K.KERNEL_GEMM
        if self._force_gemv:
            return K.KERNEL_GEMV
        if self._gemv_threshold >= 0:
            return K.KERNEL_GEMV if m <= self._gemv_threshold else K.KERNEL_GEMM
        return K.KERNEL_AUTO

    def _flatten_input(self, x: torch.Tensor):
        if x.shape[-1] != self.in_features:
            raise ValueError(f"Input dim mismatch: got {x.shape[-1]}, expected {self.in_features}")
        if not x.is_cuda:
            raise RuntimeError("CudaW4A16Linear runs on CUDA (sm_100) tensors only; there is no CPU path")
        x2d = x.reshape(-1, x.shape[-1])
        if x2d.dtype != torch.float16:
            x2d = x2d.to(torch.float16)
        return x2d.contiguous()

    def fill_member(self, mem: "K.Member", out: torch.Tensor, L: Optional[torch.Tensor] = None, alpha: float = 0.0):
        mem.qweight = self.qweight_i32.data_ptr()
        mem.scales = self.scales_f16.data_ptr()
        mem.qzeros = self.qzeros_i32.data_ptr()
        mem.bias = self.bias.data_ptr() if self.bias is not None else None
        mem.L = L.data_ptr() if L is not None else None
        mem.out = out.data_ptr()
        mem.OC = self.out_features
        mem.weight_stride_i32 = self.qweight_i32.stride(0)
        mem.zero_stride_i32 = self.qzeros_i32.stride(0)
        mem.scale_stride = self.scales_f16.stride(0)
        mem.L_stride = L.stride(0) if L is not None else 0
        mem.out_stride = out.stride(0)
        mem.alpha = float(alpha)

    def workspace_for(self, m: int, rank: int, device) -> torch.Tensor:
        key = (m, rank, device)
        if self._ws is None or self._ws_key != key:
            ext = self._get_ext()
            have = 0 if self._ws is None or self._ws.device != device else self._ws.numel()
            need = ext.workspace_bytes(m, self.in_features, self.out_features, rank, 1)
            if need > have:
                self._ws = ext.new_workspace(need, device)
            self._ws_key = key
        return self._ws

    def launch(self, x2d: torch.Tensor, *, L=None, R=None, r_buf=None, r_mode=K.R_NONE, alpha=0.0, push=None,
               push_site: int = 0) -> torch.Tensor:
        """One library call: this linear, optionally with its low-rank correction folded in.  ``push``: a
        ``glowq_b200.tp.PeerAllReduce`` - a row-split tensor-parallel shard then also stores its result into every
        rank's staging slot of ``push_site`` (complete the sum with ``push.finish(out, push_site)``)."""
        ext = self._get_ext()
        m = x2d.size(0)
        out = torch.empty((m, self.out_features), dtype=self._out_dtype, device=x2d.device)
        if m == 0:
            return out
        rank = 0 if r_mode == K.R_NONE else int(L.size(1))
        grp = K.Group()
        grp.x = x2d.data_ptr()
        grp.M, grp.IC, grp.x_stride = m, self.in_features, x2d.stride(0)
        grp.group_size = self.group_size
        grp.rank, grp.r_mode = rank, r_mode
        if r_mode != K.R_NONE:
            grp.R = R.data_ptr() if R is not None else None
            grp.R_stride = R.stride(0) if R is not None else 0
            grp.r_buf = r_buf.data_ptr()
        grp.out_dtype = K.OUT_F32 if self._out_dtype == torch.float32 else K.OUT_F16
        grp.kernel = self.kernel_choice(m)
        grp.n_members = 1
        if push is not None:
            grp.push, grp.push_site = push.descriptor_address(), int(push_site)
        self.fill_member(grp.members[0], out, L if r_mode != K.R_NONE else None, alpha)
        with torch.cuda.device(x2d.device):
            ws = self.workspace_for(m, rank, x2d.device)
            grp.workspace, grp.workspace_bytes = ws.data_ptr(), ws.numel()
            grp.stream = torch.cuda.current_stream(x2d.device).cuda_stream
            ext.check(ext.lib.glowq_w4a16_group_forward(grp), "glowq_w4a16_group_forward")
            if self._check_status:   # debugging aid: synchronises the stream after every launch
                ext.check(ext.lib.glowq_w4a16_read_status(grp.workspace, grp.stream), "device status")
        return out

    # ------------------------------------------------------------------ reference-named entry points
    def _run_cuda_gemv(self, x2d: torch.Tensor) -> torch.Tensor:
        return self._get_ext().w4a16_gemv_forward_cuda(x2d, self.qweight_i32, self.scales_f16, self.qzeros_i32,
                                                       int(self.group_size))

    def _run_cuda_gemm(self, x2d: torch.Tensor) -> torch.Tensor:
        return self._get_ext().w4a16_gemm_forward_cuda(x2d, self.qweight_i32, self.scales_f16, self.qzeros_i32,
                                                       int(self.group_size), _env_int("W4A16_SPLIT_K_ITERS", default=1))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        out = self.launch(self._flatten_input(x))
        return out.reshape(*lead, self.out_features)

    def _dequant_full_weight_fallback(self) -> torch.Tensor:
        """[OC, in_features] fp16 dequantised weight (bit-exact with linear.py:240-253), on the device."""
        return self._get_ext().dequant(self.qweight_i32, self.scales_f16, self.qzeros_i32, self.in_features,
                                       self.group_size)

    @classmethod
    def from_float(cls, linear_layer: nn.Linear, group_size: int):
        dev = linear_layer.weight.device
        mod = cls(linear_layer.in_features, linear_layer.out_features, group_size,
                  bias=linear_layer.bias is not None).to(dev)
        qw, qz, sc, _ = _quantize_per_group_w4(linear_layer.weight.data.to(torch.float16), group_size)
        for name, val in (("qweight_i32", qw), ("qzeros_i32", qz), ("scales_f16", sc)):
            buf = getattr(mod, name)
            buf.resize_(val.shape)
            buf.copy_(val)
        if linear_layer.bias is not None:
            mod.bias.data.copy_(linear_layer.bias.data.to(torch.float16))
        return mod


def convert_to_cuda_w4a16(model: nn.Module, group_size: int = 128) -> nn.Module:
    """Replace every ``nn.Linear`` whose qualified name does not contain "lm_head" (linear.py:279-293).
    A layer whose conversion raises keeps its original module, as in the reference; the failures are
    collected in ``model._w4a16_conversion_errors`` instead of vanishing."""
    errors = {}
    targets = [(n, m) for n, m in model.named_modules() if isinstance(m, nn.Linear) and "lm_head" not in n]
    for name, lin in targets:
        parent = model
        *path, leaf = name.split(".")
        for part in path:
            parent = getattr(parent, part)
        try:
            setattr(parent, leaf, CudaW4A16Linear.from_float(lin, group_size))
        except Exception as exc:  # noqa: BLE001 - parity with the reference's keep-going behaviour
            errors[name] = repr(exc)
    try:
        model._w4a16_conversion_errors = errors
    except Exception:  # noqa: BLE001
        pass
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return model
