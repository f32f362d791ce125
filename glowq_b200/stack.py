"""Synthetic decoder-stack workload for the corrected W4A16 linears (the callers of the hot path).

A ``LinearStack`` holds, for every layer of a Llama/Qwen-shaped decoder, the seven quantised projections with their
GlowQ factors (shared R for the q/k/v group and the gate/up group, own R for o_proj and down_proj), and issues one
token step of all of them through ``glowq_w4a16_group_forward_many``: four launches per layer (qkv group, o_proj,
gate/up group, down_proj) or seven when ``fuse_groups`` is off (the wrapper protocol: q computes r, k and v load it).
Weights are random-initialised and quantised with the package's own RTN quantiser; no checkpoint is involved."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .cuda_w4a16 import kernels as K
from .cuda_w4a16.linear import _quantize_per_group_w4


@dataclass
class StackShape:
    name: str
    layers: int
    hidden: int
    inter: int
    n_heads: int
    n_kv: int
    head_dim: int = 128
    rank: int = 64
    qkv_bias: bool = False
    vocab: int = 32000

    @property
    def q_out(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_out(self) -> int:
        return self.n_kv * self.head_dim


SHAPES: Dict[str, StackShape] = {
    "opt-1.3b-qkv": StackShape("opt-1.3b-qkv", 1, 2048, 8192, 32, 32, 64, 64, vocab=50272),
    "llama-3.2-3b": StackShape("llama-3.2-3b", 28, 3072, 8192, 24, 8, 128, 64, vocab=128256),
    "qwen2.5-7b": StackShape("qwen2.5-7b", 28, 3584, 18944, 28, 4, 128, 128, qkv_bias=True, vocab=152064),
    "llama-2-13b": StackShape("llama-2-13b", 40, 5120, 13824, 40, 40, 128, 128, vocab=32000),
    "qwen3-14b": StackShape("qwen3-14b", 40, 5120, 17408, 40, 8, 128, 256, vocab=151936),
}


class QLinear:
    """Device-resident packed weight + factors of one projection."""

    def __init__(self, oc: int, ic: int, rank: int, gen: torch.Generator, device, bias: bool = False, group_size=128):
        w = (torch.randn(oc, ic, generator=gen, device=device, dtype=torch.float32) * 0.02).to(torch.float16)
        self.qweight, self.qzeros, self.scales, _ = _quantize_per_group_w4(w, group_size)
        del w
        self.oc, self.ic, self.group_size = oc, ic, group_size
        self.bias = (torch.randn(oc, generator=gen, device=device) * 0.1).to(torch.float16) if bias else None
        self.L = (torch.randn(oc, rank, generator=gen, device=device) * 0.01).to(torch.float16) if rank else None

    def weight_bytes(self, corrected: bool) -> int:
        n = self.qweight.numel() * 4 + self.scales.numel() * 2 + self.qzeros.numel() * 4
        if self.bias is not None:
            n += self.oc * 2
        if corrected and self.L is not None:
            n += self.L.numel() * 2
        return n


@dataclass
class GroupSpec:
    """Projections that share an input and a right factor."""
    key: str
    members: List[QLinear]
    R: Optional[torch.Tensor]
    input_name: str                       # "hidden" or "inter"
    enabled: bool = True                  # GlowQ-S mask
    outs: List[torch.Tensor] = field(default_factory=list)
    r_buf: Optional[torch.Tensor] = None
    ws: Optional[torch.Tensor] = None


class LinearStack:
    def __init__(self, shape: StackShape, device="cuda", seed: int = 0, layers: Optional[int] = None,
                 enabled_groups: Optional[set] = None, tp_rank: int = 0, tp_world: int = 1):
        self.shape, self.device = shape, torch.device(device)
        self.ext = K.load_w4a16_extension()
        self.tp_rank, self.tp_world = tp_rank, tp_world
        gen = torch.Generator(device=self.device).manual_seed(seed + 1000 * tp_rank)
        s, r = shape, shape.rank
        n_layers = layers if layers is not None else s.layers
        tp = tp_world
        if s.q_out % tp or s.kv_out % tp or (s.inter // 128) < tp:
            raise ValueError(f"{s.name} does not shard over {tp} ranks")
        self.inter_local = self._row_shard_cols(s.inter, tp, tp_rank)
        self.attn_local = s.q_out // tp
        self.groups: List[GroupSpec] = []

        def fac(rows, cols):
            return (torch.randn(rows, cols, generator=gen, device=self.device) * 0.01).to(torch.float16)

        for li in range(n_layers):
            def on(key):
                return enabled_groups is None or key in enabled_groups
            qkv = [QLinear(s.q_out // tp, s.hidden, r, gen, self.device, s.qkv_bias),
                   QLinear(s.kv_out // tp, s.hidden, r, gen, self.device, s.qkv_bias),
                   QLinear(s.kv_out // tp, s.hidden, r, gen, self.device, s.qkv_bias)]
            self.groups.append(GroupSpec(f"layer{li}_qkv", qkv, fac(r, s.hidden), "hidden", on(f"layer{li}_qkv")))
            o = QLinear(s.hidden, self.attn_local, r, gen, self.device)
            k = f"model.layers.{li}.self_attn.o_proj"
            self.groups.append(GroupSpec(k, [o], fac(r, self.attn_local), "attn", on(k)))
            mlp = [QLinear(self.inter_local, s.hidden, r, gen, self.device) for _ in range(2)]
            self.groups.append(GroupSpec(f"layer{li}_mlp", mlp, fac(r, s.hidden), "hidden", on(f"layer{li}_mlp")))
            d = QLinear(s.hidden, self.inter_local, r, gen, self.device)
            k = f"model.layers.{li}.mlp.down_proj"
            self.groups.append(GroupSpec(k, [d], fac(r, self.inter_local), "inter", on(k)))
        self._plans = {}

    @staticmethod
    def _row_shard_cols(cols: int, world: int, rank: int, group: int = 128) -> int:
        """Input columns of a row-split linear on ``rank``: whole quantisation groups, the first
        ``G % world`` ranks taking one group more (13824 over 8 ranks -> 4 x 1792 + 4 x 1664)."""
        g = cols // group
        return (g // world + (1 if rank < g % world else 0)) * group

    # ------------------------------------------------------------------ bytes / flops (algorithmic)
    def algorithmic_bytes(self, M: int, corrected: bool = True) -> int:
        total = 0
        for g in self.groups:
            use = corrected and g.enabled
            for m in g.members:
                total += m.weight_bytes(use) + M * m.oc * 2
            total += M * g.members[0].ic * 2
            if use:
                total += g.R.numel() * 2
        return total

    def algorithmic_flops(self, M: int, corrected: bool = True) -> int:
        total = 0
        for g in self.groups:
            use = corrected and g.enabled
            for m in g.members:
                total += 2 * M * m.oc * m.ic + (2 * M * m.oc * self.shape.rank if use else 0)
            if use:
                total += 2 * M * self.shape.rank * g.members[0].ic
        return total

    # ------------------------------------------------------------------ launch plans
    def plan(self, M: int, *, corrected: bool = True, fuse_groups: bool = True, kernel: int = K.KERNEL_AUTO,
             out_dtype: int = K.OUT_F16, split_k: int = 0):
        """Build (once per configuration) the ctypes array of group calls for one token step of M tokens."""
        key = (M, corrected, fuse_groups, kernel, out_dtype, split_k)
        if key in self._plans:
            return self._plans[key]
        s = self.shape
        dt = torch.float16 if out_dtype == K.OUT_F16 else torch.float32
        gen = torch.Generator(device=self.device).manual_seed(2)
        inputs = {"hidden": torch.randn(M, s.hidden, generator=gen, device=self.device).to(torch.float16),
                  "attn": torch.randn(M, self.attn_local, generator=gen, device=self.device).to(torch.float16),
                  "inter": torch.randn(M, self.inter_local, generator=gen, device=self.device).to(torch.float16)}
        calls = []
        keep = [inputs]
        stream = torch.cuda.current_stream(self.device).cuda_stream
        for g in self.groups:
            outs = [torch.empty(M, m.oc, dtype=dt, device=self.device) for m in g.members]
            r_buf = torch.zeros(max(M, 1), s.rank, dtype=torch.float16, device=self.device)
            use = corrected and g.enabled
            member_sets = [g.members] if fuse_groups else [[m] for m in g.members]
            off = 0
            for si, ms in enumerate(member_sets):
                need = self.ext.workspace_bytes(M, ms[0].ic, sum(m.oc for m in ms), s.rank if use else 0, len(ms))
                ws = self.ext.new_workspace(need + (32 << 20 if split_k else 0), self.device)
                c = K.Group()
                x = inputs[g.input_name]
                c.x, c.M, c.IC, c.x_stride = x.data_ptr(), M, ms[0].ic, x.stride(0)
                c.group_size = ms[0].group_size
                c.out_dtype, c.kernel, c.split_k = out_dtype, kernel, split_k
                if use:
                    c.rank = s.rank
                    c.r_mode = K.R_COMPUTE if si == 0 else K.R_LOAD
                    c.R, c.R_stride = g.R.data_ptr(), g.R.stride(0)
                    c.r_buf = r_buf.data_ptr()
                c.n_members = len(ms)
                for i, m in enumerate(ms):
                    mem = c.members[i]
                    o = outs[off + i]
                    mem.qweight, mem.scales, mem.qzeros = m.qweight.data_ptr(), m.scales.data_ptr(), m.qzeros.data_ptr()
                    mem.bias = m.bias.data_ptr() if m.bias is not None else None
                    if use:
                        mem.L, mem.L_stride = m.L.data_ptr(), m.L.stride(0)
                    mem.out, mem.out_stride, mem.OC = o.data_ptr(), o.stride(0), m.oc
                    mem.weight_stride_i32, mem.zero_stride_i32 = m.qweight.stride(0), m.qzeros.stride(0)
                    mem.scale_stride = m.scales.stride(0)
                    mem.alpha = 1.0
                off += len(ms)
                c.workspace, c.workspace_bytes, c.stream = ws.data_ptr(), ws.numel(), stream
                calls.append(c)
                keep.append(ws)
            keep += [outs, r_buf]
        arr = (K.Group * len(calls))(*calls)
        plan = {"calls": arr, "n": len(calls), "inputs": inputs, "keep": keep,
                "last_out": keep[-2][-1], "M": M}
        self._plans[key] = plan
        return plan

    def step(self, plan) -> None:
        """Enqueue one token step (no synchronisation)."""
        self.ext.check(self.ext.lib.glowq_w4a16_group_forward_many(plan["calls"], plan["n"]), "group_forward_many")

    def check_status(self, plan) -> None:
        stream = torch.cuda.current_stream(self.device).cuda_stream
        for c in plan["calls"]:
            self.ext.check(self.ext.lib.glowq_w4a16_read_status(c.workspace, stream), "device status")
