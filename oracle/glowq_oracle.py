"""CPU restatement of GlowQ's corrected W4A16 linear (TEST INFRASTRUCTURE ONLY).

This module is the checker for the CUDA path: tests, the smoke entry and the
CPU-baseline leg of the benchmark may import it; the product package never does.

It restates, in numpy, the arithmetic of the reference's Python path:

* RTN asymmetric uint4 quantiser and int32 packer
  (src/cuda_w4a16/linear.py:42-46, 57-88),
* the unpack + dequantise definition ``half((code - zero) * scale)``
  (src/cuda_w4a16/linear.py:49-54, 248-253; csrc/gemm_w4a16.cu:44-49),
* the corrected forward ``y = x . dequant(Q)^T + alpha * (x . R^T) . L^T + bias``
  (src/cuda_w4a16/linear.py:155-187 + src/step3_eval_dataset.py:470-511)
  evaluated in fp32, which is the result the parity tolerances are quoted against,
* the shared-right-factor cache protocol (src/step3_eval_dataset.py:417-444, 481-504).

Parity pin: every function here is checked against outputs of the reference's own
code (imported in place and run on seeded inputs) stored under tests/golden/ by
tests/golden/make_golden.py.  The reference itself ships no golden vectors.
"""
from __future__ import annotations

import numpy as np

__all__ = [
    "pack_int4_to_int32",
    "unpack_int4_i32",
    "quantize_per_group_w4",
    "dequant_full",
    "plain_forward_fp32",
    "corrected_forward_fp32",
    "reference_rounded_forward",
    "GroupCacheModel",
    "role_from_suffix",
    "parity_errors",
]


def pack_int4_to_int32(u4: np.ndarray) -> np.ndarray:
    """Pack the last axis (length 8) of uint8 codes into one int32, nibble i at
    bits [4i, 4i+4) (src/cuda_w4a16/linear.py:42-46).  A top nibble >= 8 wraps
    to a negative word, as int32 addition does in the reference."""
    assert u4.dtype == np.uint8 and u4.shape[-1] == 8
    shifts = (np.arange(8, dtype=np.uint32) * 4)
    word = (u4.astype(np.uint32) << shifts).sum(axis=-1, dtype=np.uint32)
    return word.view(np.int32)


def unpack_int4_i32(packed: np.ndarray, total_vals: int) -> np.ndarray:
    """Inverse of the packer, row-wise, truncated to ``total_vals`` columns
    (src/cuda_w4a16/linear.py:49-54)."""
    p = np.ascontiguousarray(packed).view(np.uint32)
    rows = p.shape[0]
    shifts = (np.arange(8, dtype=np.uint32) * 4).reshape(1, 1, 8)
    vals = ((p[..., None] >> shifts) & 0xF).astype(np.uint8)
    return np.ascontiguousarray(vals.reshape(rows, -1)[:, :total_vals])


def quantize_per_group_w4(weight_f16: np.ndarray, group_size: int):
    """RTN asymmetric uint4 per (row, group) in fp16 arithmetic
    (src/cuda_w4a16/linear.py:57-88).

    Returns (qweight_i32 [OC, ICp/8], qzeros_i32 [OC, ceil(G/8)], scales_f16 [OC, G], ICp).
    fp16 arithmetic makes ``clamp(min=1e-8)`` a no-op (1e-8 rounds to 0 in fp16), so a
    constant group has scale 0; the resulting inf/NaN follow IEEE rules and NaN casts to
    code 0, which is what the reference produces on x86."""
    w = np.asarray(weight_f16)
    assert w.dtype == np.float16 and w.ndim == 2
    if group_size <= 0 or group_size % 8 != 0:
        raise ValueError("group_size must be multiple of 8 for int32 int4 packing")
    oc, ic = w.shape
    if ic % group_size != 0:
        pad = group_size - ic % group_size
        w = np.pad(w, ((0, 0), (0, pad)))
        ic = w.shape[1]
    groups = ic // group_size
    wg = w.reshape(oc, groups, group_size)
    with np.errstate(all="ignore"):
        w_min = wg.min(axis=-1)
        w_max = wg.max(axis=-1)
        scales = np.maximum(((w_max - w_min) / np.float16(15.0)).astype(np.float16), np.float16(1e-8))
        zeros_fp = np.clip(np.rint((-w_min / scales).astype(np.float16)), 0, 15)
        qf = (wg / scales[..., None]).astype(np.float16) + zeros_fp[..., None].astype(np.float16)
        qf = np.clip(np.rint(qf.astype(np.float16)), 0, 15)
    q = np.nan_to_num(qf.astype(np.float32), nan=0.0).astype(np.uint8)
    zeros_u8 = np.nan_to_num(zeros_fp.astype(np.float32), nan=0.0).astype(np.uint8)

    q_packed = pack_int4_to_int32(q.reshape(oc, groups, group_size // 8, 8)).reshape(oc, ic // 8)
    groups_packed = (groups + 7) // 8
    zeros_base = np.pad(zeros_u8, ((0, 0), (0, groups_packed * 8 - groups)), constant_values=8)
    zeros_packed = pack_int4_to_int32(zeros_base.reshape(oc, groups_packed, 8))
    return (np.ascontiguousarray(q_packed), np.ascontiguousarray(zeros_packed),
            np.ascontiguousarray(scales.astype(np.float16)), ic)


def dequant_full(qweight_i32, qzeros_i32, scales_f16, in_features: int, group_size: int) -> np.ndarray:
    """fp16 weight ``(code - zero) * scale`` with one fp16 rounding of the product
    (src/cuda_w4a16/linear.py:248-253).  ``code - zero`` is an exact small integer and the
    product is exact in fp32, so rounding it once equals csrc/gemm_w4a16.cu:46-49."""
    groups = -(-in_features // group_size)
    groups_packed = (groups + 7) // 8
    gid = np.arange(in_features) // group_size
    qv = unpack_int4_i32(qweight_i32, in_features).astype(np.float32)
    zv = unpack_int4_i32(qzeros_i32[:, :max(1, groups_packed)], groups).astype(np.float32)
    sc = np.asarray(scales_f16)[:, :groups].astype(np.float32)
    return ((qv - zv[:, gid]) * sc[:, gid]).astype(np.float16)


def plain_forward_fp32(x_f16, w_deq_f16, bias_f16=None) -> np.ndarray:
    """``x.float() @ dequant(Q).float().T (+ bias)``: the uncorrected W4A16 linear in fp32."""
    y = np.asarray(x_f16, dtype=np.float32) @ np.asarray(w_deq_f16, dtype=np.float32).T
    if bias_f16 is not None:
        y = y + np.asarray(bias_f16, dtype=np.float32)
    return y


def corrected_forward_fp32(x_f16, w_deq_f16, R_f16=None, L_f16=None, alpha: float = 1.0, bias_f16=None):
    """fp32 oracle of ``AddSVDCorrection(CudaW4A16Linear)``: the inner linear including its bias
    (src/cuda_w4a16/linear.py:183-187) plus ``alpha * (x R^T) L^T`` (src/step3_eval_dataset.py:470-511).
    ``alpha == 0`` or missing factors give the plain linear (step3_eval_dataset.py:473-474)."""
    y = plain_forward_fp32(x_f16, w_deq_f16, bias_f16)
    if R_f16 is None or L_f16 is None or alpha == 0.0:
        return y
    x32 = np.asarray(x_f16, dtype=np.float32)
    r = x32 @ np.asarray(R_f16, dtype=np.float32).T
    return y + np.float32(alpha) * (r @ np.asarray(L_f16, dtype=np.float32).T)


def reference_rounded_forward(x_f16, w_deq_f16, R_f16, L_f16, alpha: float = 1.0, bias_f16=None,
                              out_dtype=np.float16):
    """The reference module path with its intermediate roundings, for reading the golden
    ``y_ref`` fixtures: matmul result -> out dtype, + bias, ``r`` and ``L r`` each rounded to
    fp16 by ``F.linear`` (step3_eval_dataset.py:484, 506), then the in-place add in the out
    dtype (:511).  Accumulation order inside the matmuls is the library's, so this agrees with
    the reference only to accumulation rounding, not bitwise."""
    z = (np.asarray(x_f16, np.float32) @ np.asarray(w_deq_f16, np.float32).T).astype(np.float16)
    z = z.astype(out_dtype)
    if bias_f16 is not None:
        z = (z + np.asarray(bias_f16).astype(out_dtype)).astype(out_dtype)
    if alpha == 0.0:
        return z
    r = (np.asarray(x_f16, np.float32) @ np.asarray(R_f16, np.float32).T).astype(np.float16)
    c = (r.astype(np.float32) @ np.asarray(L_f16, np.float32).T).astype(np.float16)
    return (z.astype(np.float32) + np.float32(alpha) * c.astype(np.float32)).astype(out_dtype)


def role_from_suffix(sfx: str) -> str:
    """Module-name suffix -> cache role (src/step3_eval_dataset.py:519-532)."""
    for end, role in (("q_proj", "q"), ("k_proj", "k"), ("v_proj", "v"),
                      ("gate_proj", "gate"), ("up_proj", "up")):
        if sfx.endswith(end):
            return role
    return "solo"


class GroupCacheModel:
    """State machine of ``MiniGroupCache`` plus the role logic of ``AddSVDCorrection.forward``
    (src/step3_eval_dataset.py:417-444, 481-504).  ``step(role)`` returns "compute" when the
    wrapper evaluates ``R x`` itself and "hit" when it consumes the cached product."""

    def __init__(self):
        self.valid = False
        self.uses_left = 0

    def step(self, role: str, is_group: bool = True) -> str:
        if not is_group or role not in ("q", "gate", "k", "v", "up"):
            return "compute"
        if role in ("q", "gate"):
            self.valid, self.uses_left = True, (2 if role == "q" else 1)
            return "compute"
        if self.valid and self.uses_left > 0:
            self.uses_left -= 1
            if self.uses_left == 0:
                self.valid = False
            return "hit"
        return "compute"


def residual_rmsnorm_f16(x_f16, residual_f16, weight_f16, eps: float):
    """The residual add and RMSNorm that precede q/k/v and gate/up in a Llama / Qwen decoder block, as the model code
    the reference runs computes them (the reference itself has no norm code: it evaluates HF models, whose
    ``LlamaRMSNorm.forward`` - transformers models/llama/modeling_llama.py - and decoder layer do exactly this):
        h  = residual + x                          fp16 add (one rounding)
        xn = weight * (h.float() * rsqrt(mean(h.float()^2) + eps)).half()      fp16 product (one more rounding)
    Returns (xn fp16, h fp16)."""
    x = np.asarray(x_f16, dtype=np.float16)
    h = x if residual_f16 is None else (x.astype(np.float32) + np.asarray(residual_f16, np.float16).astype(np.float32)
                                        ).astype(np.float16)
    hf = h.astype(np.float32)
    var = np.mean(hf * hf, axis=-1, keepdims=True, dtype=np.float32)
    n = (hf * (1.0 / np.sqrt(var + np.float32(eps))).astype(np.float32)).astype(np.float16)
    xn = (np.asarray(weight_f16, np.float16).astype(np.float32) * n.astype(np.float32)).astype(np.float16)
    return xn, h


def parity_errors(y, y_ref):
    """(max-abs error, mean-rel error) with mean-rel = mean|y - y_ref| / mean|y_ref|."""
    y = np.asarray(y, dtype=np.float64)
    y_ref = np.asarray(y_ref, dtype=np.float64)
    if y.size == 0:
        return 0.0, 0.0
    d = np.abs(y - y_ref)
    return float(d.max()), float(d.mean() / max(np.abs(y_ref).mean(), 1e-30))
