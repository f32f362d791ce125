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

    def as_module(self):
        """A ``CudaW4A16Linear`` shell over the same packed tensors (what ``glowq_b200.tp`` shards)."""
        from .cuda_w4a16.linear import CudaW4A16Linear
        mod = CudaW4A16Linear(self.ic, self.oc, self.group_size, bias=self.bias is not None).to(self.qweight.device)
        for name, t in (("qweight_i32", self.qweight), ("qzeros_i32", self.qzeros), ("scales_f16", self.scales)):
            buf = getattr(mod, name)
            buf.resize_(t.shape)
            buf.copy_(t)
        if self.bias is not None:
            mod.bias.data.copy_(self.bias)
        return mod

    @classmethod
    def from_module(cls, mod, L):
        """The other direction: a (sharded) module and its left factor as a ``QLinear``."""
        q = cls.__new__(cls)
        q.qweight, q.qzeros, q.scales = (mod.qweight_i32.contiguous(), mod.qzeros_i32.contiguous(),
                                         mod.scales_f16.contiguous())
        q.oc, q.ic, q.group_size = mod.out_features, mod.in_features, mod.group_size
        q.bias = None if mod.bias is None else mod.bias.data.contiguous()
        q.L = None if L is None else L.contiguous()
        return q

    def numpy_parts(self):
        return {"qweight": self.qweight.cpu().numpy(), "qzeros": self.qzeros.cpu().numpy(),
                "scales": self.scales.cpu().numpy(), "L": None if self.L is None else self.L.cpu().numpy(),
                "bias": None if self.bias is None else self.bias.cpu().numpy()}

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
    """``tp_world`` > 1: every rank draws the SAME full model from ``seed`` and keeps its tensor-parallel shard, cut by
    ``glowq_b200.tp``: q/k/v and gate/up by output rows (whole heads / whole 128-row blocks, R replicated), o_proj and
    down_proj by input columns at quantisation-group boundaries (R cut with them, L replicated).  The partial outputs
    of the row-split members add up to the unsharded result; ``tp_reference`` keeps layer 0's unsharded o_proj and
    down_proj (numpy) so that a caller can check that sum."""

    def __init__(self, shape: StackShape, device="cuda", seed: int = 0, layers: Optional[int] = None,
                 enabled_groups: Optional[set] = None, tp_rank: int = 0, tp_world: int = 1):
        from . import tp as TP
        self.shape, self.device = shape, torch.device(device)
        self.ext = K.load_w4a16_extension()
        self.tp_rank, self.tp_world = tp_rank, tp_world
        gen = torch.Generator(device=self.device).manual_seed(seed)     # same stream of draws on every rank
        s, r = shape, shape.rank
        n_layers = layers if layers is not None else s.layers
        tp = tp_world
        if tp > 1 and (s.q_out % (tp * s.head_dim) or s.kv_out % (tp * s.head_dim) or (s.inter // 128) < tp
                       or s.head_dim % 128):
            raise ValueError(f"{s.name} does not shard over {tp} ranks")
        # input-column ranges of the row-split members on this rank (whole quantisation groups)
        a0, a1 = [(g0 * 128, g1 * 128) for g0, g1 in TP.group_bounds(s.q_out // 128, tp)][tp_rank]
        i0, i1 = [(g0 * 128, g1 * 128) for g0, g1 in TP.group_bounds(s.inter // 128, tp)][tp_rank]
        self.attn_cols, self.inter_cols = (a0, a1), (i0, i1)
        self.inter_local, self.attn_local = i1 - i0, a1 - a0
        self.groups: List[GroupSpec] = []
        self.tp_reference: Dict[str, dict] = {}

        def fac(rows, cols):
            return (torch.randn(rows, cols, generator=gen, device=self.device) * 0.01).to(torch.float16)

        def col_shard(full: QLinear, multiple: int) -> QLinear:
            if tp == 1:
                return full
            sh, L_sh = TP.column_parallel_shard(full.as_module(), tp_rank, tp, multiple=multiple, L=full.L)
            return QLinear.from_module(sh, L_sh)

        def row_shard(full: QLinear, R: torch.Tensor, key: str, li: int):
            if tp == 1:
                return full, R
            if li == 0 and tp_rank == 0:
                self.tp_reference[key] = dict(full.numpy_parts(), R=R.cpu().numpy())
            sh, R_sh, _ = TP.row_parallel_shard(full.as_module(), tp_rank, tp, R=R)
            return QLinear.from_module(sh, full.L), R_sh

        for li in range(n_layers):
            def on(key):
                return enabled_groups is None or key in enabled_groups
            qkv = [col_shard(QLinear(oc, s.hidden, r, gen, self.device, s.qkv_bias), s.head_dim)
                   for oc in (s.q_out, s.kv_out, s.kv_out)]
            self.groups.append(GroupSpec(f"layer{li}_qkv", qkv, fac(r, s.hidden), "hidden", on(f"layer{li}_qkv")))
            k = f"model.layers.{li}.self_attn.o_proj"
            o, R_o = row_shard(QLinear(s.hidden, s.q_out, r, gen, self.device), fac(r, s.q_out), "o_proj", li)
            self.groups.append(GroupSpec(k, [o], R_o, "attn", on(k)))
            mlp = [col_shard(QLinear(s.inter, s.hidden, r, gen, self.device), 128) for _ in range(2)]
            self.groups.append(GroupSpec(f"layer{li}_mlp", mlp, fac(r, s.hidden), "hidden", on(f"layer{li}_mlp")))
            k = f"model.layers.{li}.mlp.down_proj"
            d, R_d = row_shard(QLinear(s.hidden, s.inter, r, gen, self.device), fac(r, s.inter), "down_proj", li)
            self.groups.append(GroupSpec(k, [d], R_d, "inter", on(k)))
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
             out_dtype: int = K.OUT_F16, split_k: int = 0, chain: bool = True, push=None):
        """Build (once per configuration) the ctypes array of group calls for one token step of M tokens."""
        # push: a glowq_b200.tp.PeerAllReduce - the row-split groups (o_proj, down_proj) then store their partial result
        # into every rank's staging slot themselves (sites alternate) and write the sum over the ranks to their output
        key = (M, corrected, fuse_groups, kernel, out_dtype, split_k, chain, id(push))
        if key in self._plans:
            return self._plans[key]
        s = self.shape
        dt = torch.float16 if out_dtype == K.OUT_F16 else torch.float32
        gen = torch.Generator(device=self.device).manual_seed(2)
        full = {"hidden": torch.randn(M, s.hidden, generator=gen, device=self.device).to(torch.float16),
                "attn": torch.randn(M, s.q_out, generator=gen, device=self.device).to(torch.float16),
                "inter": torch.randn(M, s.inter, generator=gen, device=self.device).to(torch.float16)}
        # every rank draws the same full activations and keeps the columns its row-split members consume
        inputs = {"hidden": full["hidden"],
                  "attn": full["attn"][:, self.attn_cols[0]:self.attn_cols[1]].contiguous(),
                  "inter": full["inter"][:, self.inter_cols[0]:self.inter_cols[1]].contiguous()}
        calls = []
        keep = [inputs]
        group_outs = []
        n_row_split = 0
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
                if push is not None and g.input_name in ("attn", "inter") and len(ms) == 1 and M <= 8 \
                        and out_dtype == K.OUT_F16:
                    c.push, c.push_site = push.descriptor_address(), n_row_split & 1
                    n_row_split += 1
                c.workspace, c.workspace_bytes, c.stream = ws.data_ptr(), ws.numel(), stream
                calls.append(c)
                keep.append(ws)
            keep += [outs, r_buf]
            group_outs.append(outs)
        arr = (K.Group * len(calls))(*calls)
        if chain:   # tell every call what follows it on the stream (the last one: the next step's first call)
            for i in range(len(calls)):
                arr[i].next = ctypes.addressof(arr[(i + 1) % len(calls)])
        plan = {"calls": arr, "n": len(calls), "inputs": inputs, "full_inputs": full, "keep": keep,
                "last_out": keep[-2][-1], "M": M, "group_outs": group_outs}
        self._plans[key] = plan
        return plan

    def step(self, plan) -> None:
        """Enqueue one token step (no synchronisation)."""
        self.ext.check(self.ext.lib.glowq_w4a16_group_forward_many(plan["calls"], plan["n"]), "group_forward_many")

    def check_status(self, plan) -> None:
        stream = torch.cuda.current_stream(self.device).cuda_stream
        for c in plan["calls"]:
            self.ext.check(self.ext.lib.glowq_w4a16_read_status(c.workspace, stream), "device status")
