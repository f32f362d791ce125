"""Packed checkpoints: write the converted model's int4 weights once, reload them without re-quantising.

The reference re-runs ``convert_to_cuda_w4a16`` (an fp16 RTN quantisation of every linear) at the start of every
step3 / step4 run, and once per cumulative point of the GlowQ-S sweep
(src/restoration/step4_evaluate_cumulative.py:173-184).  The packed tensors are deterministic functions of the fp16
weights, so they can be stored next to the low-rank artefacts and loaded straight into ``CudaW4A16Linear`` shells.

File layout (one ``torch.save`` dict, tensors on CPU):
  ``format``: "glowq_b200.packed.v1"
  ``group_size``: int
  ``modules``: {qualified module name: {"in_features", "out_features", "bias": bool}}
  ``tensors``: {"<name>.qweight_i32" [OC, ICp/8] int32, "<name>.qzeros_i32" [OC, ceil(G/8)] int32,
                "<name>.scales_f16" [OC, G] fp16, "<name>.bias" [OC] fp16 (if any)}   - the module's own buffer names
  ``low_rank``: optional {"shared": dict as in low_rank_shared.pt (src/step2_rsvd.py:487-522), "bmap": b_ref_map.json}
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from .cuda_w4a16.linear import CudaW4A16Linear

FORMAT = "glowq_b200.packed.v1"
_BUFFERS = ("qweight_i32", "qzeros_i32", "scales_f16")


def _unwrap(mod: nn.Module) -> nn.Module:
    """The packed linear inside a correction wrapper (wrappers keep it as ``.inner``)."""
    inner = getattr(mod, "inner", None)
    return inner if isinstance(inner, CudaW4A16Linear) else mod


def packed_state(model: nn.Module) -> Tuple[Dict[str, dict], Dict[str, torch.Tensor], Optional[int]]:
    """(modules, tensors, group_size) of every ``CudaW4A16Linear`` in ``model`` (wrapped or bare), keyed by the name
    the module has in the un-patched model."""
    modules, tensors, gs = {}, {}, None
    for name, mod in model.named_modules():
        if name.endswith(".inner"):
            continue  # reached through its wrapper, under the wrapper's name
        lin = _unwrap(mod)
        if not isinstance(lin, CudaW4A16Linear):
            continue
        if gs is None:
            gs = int(lin.group_size)
        elif gs != int(lin.group_size):
            raise ValueError(f"{name}: group size {lin.group_size} differs from {gs}")
        modules[name] = {"in_features": int(lin.in_features), "out_features": int(lin.out_features),
                         "bias": lin.bias is not None}
        for b in _BUFFERS:
            tensors[f"{name}.{b}"] = getattr(lin, b).detach().to("cpu").contiguous()
        if lin.bias is not None:
            tensors[f"{name}.bias"] = lin.bias.detach().to("cpu", torch.float16).contiguous()
    return modules, tensors, gs


def save_packed(model: nn.Module, path: str, shared: Optional[Dict[str, torch.Tensor]] = None,
                bmap: Optional[Dict[str, str]] = None) -> int:
    """Write the packed weights of ``model`` (and, if given, the low-rank artefacts) to ``path``.
    Returns the number of packed modules."""
    modules, tensors, gs = packed_state(model)
    if not modules:
        raise ValueError("the model holds no CudaW4A16Linear module: run convert_to_cuda_w4a16 first")
    blob = {"format": FORMAT, "group_size": gs, "modules": modules, "tensors": tensors}
    if shared is not None or bmap is not None:
        blob["low_rank"] = {"shared": {k: v.detach().to("cpu") for k, v in (shared or {}).items()},
                            "bmap": dict(bmap or {})}
    torch.save(blob, path)
    return len(modules)


def load_packed(model: nn.Module, path: str, device=None, strict: bool = True):
    """Replace the ``nn.Linear`` modules of ``model`` named in the checkpoint by ``CudaW4A16Linear`` modules holding the
    stored tensors - the result equals ``convert_to_cuda_w4a16(model, group_size)`` bit for bit, without quantising.
    ``strict``: every stored module must exist in ``model`` with matching sizes, and (as in the conversion pass,
    src/cuda_w4a16/linear.py:279-293) every ``nn.Linear`` outside "lm_head" must be covered.
    Returns ``(model, shared, bmap)``; the last two are None when the file holds no low-rank artefacts."""
    blob = torch.load(path, map_location="cpu", weights_only=True)
    if not isinstance(blob, dict) or blob.get("format") != FORMAT:
        raise ValueError(f"{path}: not a {FORMAT} file")
    gs, modules, tensors = int(blob["group_size"]), blob["modules"], blob["tensors"]
    named = dict(model.named_modules())
    missing = [n for n in modules if n not in named]
    if strict and missing:
        raise KeyError(f"modules absent from the model: {missing[:4]}{'...' if len(missing) > 4 else ''}")
    if strict:
        uncovered = [n for n, m in named.items() if isinstance(m, nn.Linear) and "lm_head" not in n and n not in modules]
        if uncovered:
            raise KeyError(f"linear layers without packed weights: {uncovered[:4]}{'...' if len(uncovered) > 4 else ''}")
    for name, meta in modules.items():
        old = named.get(name)
        if old is None:
            continue
        if isinstance(old, (nn.Linear, CudaW4A16Linear)):
            if (old.in_features, old.out_features) != (meta["in_features"], meta["out_features"]):
                raise ValueError(f"{name}: stored {meta['out_features']}x{meta['in_features']}, "
                                 f"model has {old.out_features}x{old.in_features}")
        dev = device
        if dev is None:
            dev = next((t.device for t in list(old.parameters()) + list(old.buffers())), torch.device("cpu"))
        new = CudaW4A16Linear(meta["in_features"], meta["out_features"], gs, bias=meta["bias"])
        for b in _BUFFERS:
            t = tensors[f"{name}.{b}"]
            buf = getattr(new, b)
            # the stored tensors have the quantiser's shapes (columns padded to whole groups, as from_float leaves
            # them), which may be wider than the fresh shell's ceil(IC/8) columns
            if (buf.dtype != t.dtype or t.dim() != 2 or t.size(0) != buf.size(0) or t.size(1) < buf.size(1)):
                raise ValueError(f"{name}.{b}: stored {tuple(t.shape)} {t.dtype}, expected at least "
                                 f"{tuple(buf.shape)} {buf.dtype}")
            buf.resize_(t.shape)
            buf.copy_(t)
        if meta["bias"]:
            new.bias.data.copy_(tensors[f"{name}.bias"])
        new = new.to(dev)
        parent = model
        *parts, leaf = name.split(".")
        for part in parts:
            parent = getattr(parent, part)
        setattr(parent, leaf, new)
    lr = blob.get("low_rank")
    if lr is None:
        return model, None, None
    return model, lr["shared"], lr["bmap"]
