"""Tensor-parallel sharding of corrected W4A16 linears (the reference is single-GPU; this is the layout the
benchmark configurations prescribe).

* column-parallel (q, k, v, gate, up): packed weight, scales, zero words, bias and the left factor L are split by
  OUTPUT rows; the shared right factor R is replicated, so r = R x is recomputed on every rank and no collective
  is needed; the output stays sharded.
* row-parallel (o_proj, down_proj): the packed weight is split by INPUT columns at 128-column group boundaries
  (scales and zero nibbles with it - zero words are re-packed because a shard may start in the middle of a word),
  R by the same columns, L replicated.  By linearity sum_p [ Wq[:, p] x_p + L (R[:, p] x_p) ] is the corrected
  output: one all-reduce of [M, hidden] finishes the layer.  Bias is added on rank 0 only.

When the group count does not divide by the world size the first ``G % world`` ranks take one group more
(13824 columns over 8 ranks: 4 x 1792 + 4 x 1664); the matching column-parallel producer (gate / up) must be split
with the same boundaries."""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from .cuda_w4a16.linear import CudaW4A16Linear, _pack_int4_to_int32, _unpack_int4_i32


def group_bounds(n_groups: int, world: int) -> List[Tuple[int, int]]:
    """[g0, g1) of every rank: whole groups, remainder spread over the first ranks."""
    base, rem = divmod(n_groups, world)
    out, g = [], 0
    for r in range(world):
        n = base + (1 if r < rem else 0)
        out.append((g, g + n))
        g += n
    return out


def row_bounds(n_rows: int, world: int, multiple: int = 1) -> List[Tuple[int, int]]:
    """Output-row ranges of a column-parallel linear, in units of ``multiple`` rows (e.g. a head, or the 128-row
    blocks that keep a gate/up shard aligned with the row-parallel consumer's column groups)."""
    if n_rows % multiple:
        raise ValueError(f"{n_rows} rows are not a multiple of {multiple}")
    return [(a * multiple, b * multiple) for a, b in group_bounds(n_rows // multiple, world)]


def column_parallel_shard(mod: CudaW4A16Linear, rank: int, world: int, multiple: int = 1,
                          L: Optional[torch.Tensor] = None):
    """(sharded module, sharded L) holding output rows of ``rank``."""
    r0, r1 = row_bounds(mod.out_features, world, multiple)[rank]
    out = CudaW4A16Linear(mod.in_features, r1 - r0, mod.group_size, bias=mod.bias is not None)
    out = out.to(mod.qweight_i32.device)
    for name in ("qweight_i32", "qzeros_i32", "scales_f16"):
        src = getattr(mod, name)[r0:r1].contiguous()
        buf = getattr(out, name)
        buf.resize_(src.shape)
        buf.copy_(src)
    if mod.bias is not None:
        out.bias.data.copy_(mod.bias.data[r0:r1])
    return out, (None if L is None else L[r0:r1].contiguous())


def row_parallel_shard(mod: CudaW4A16Linear, rank: int, world: int, R: Optional[torch.Tensor] = None):
    """(sharded module, sharded R, (c0, c1)) holding input columns [c0, c1) of ``rank``; bias stays on rank 0."""
    gs = mod.group_size
    n_groups = mod.scales_f16.size(1)
    g0, g1 = group_bounds(n_groups, world)[rank]
    c0, c1 = g0 * gs, min(g1 * gs, max(mod.in_features, g0 * gs))
    in_local = max(0, min(mod.in_features, g1 * gs) - c0)
    keep_bias = mod.bias is not None and rank == 0
    out = CudaW4A16Linear(max(in_local, 1), mod.out_features, gs, bias=keep_bias).to(mod.qweight_i32.device)
    out.in_features = in_local
    qw = mod.qweight_i32[:, g0 * gs // 8:g1 * gs // 8].contiguous()
    sc = mod.scales_f16[:, g0:g1].contiguous()
    z = _unpack_int4_i32(mod.qzeros_i32, n_groups)[:, g0:g1]
    words = max(1, (g1 - g0 + 7) // 8)
    z = torch.nn.functional.pad(z, (0, words * 8 - (g1 - g0)), value=8)
    qz = _pack_int4_to_int32(z.view(z.size(0), words, 8)).contiguous()
    for name, src in (("qweight_i32", qw), ("qzeros_i32", qz), ("scales_f16", sc)):
        buf = getattr(out, name)
        buf.resize_(src.shape)
        buf.copy_(src)
    out.groups, out.groups_packed = g1 - g0, words
    out.gid = (torch.arange(in_local, dtype=torch.long, device=mod.gid.device) // gs)
    if keep_bias:
        out.bias.data.copy_(mod.bias.data)
    R_local = None if R is None else R[:, c0:c0 + in_local].contiguous()
    return out, R_local, (c0, c0 + in_local)


class PeerAllReduce:
    """Sum small fp16 tensors across the ranks of one node with the library's peer-store all-reduce
    (``glowq_w4a16_allreduce_f16``): no NCCL call, so the collective can sit inside a captured CUDA graph.

    Staging buffers and epoch flags live in torch symmetric memory (one allocation per rank, mapped into every peer);
    PyTorch only provides the mapping - the data movement is the library's kernel.  Two "sites" are used alternately,
    which is enough for a site never to be rewritten while a slower rank still reads it (a rank can only be two
    calls ahead of another after that rank has finished the call in between)."""

    SITES = 2

    def __init__(self, group, device, max_elems: int):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        from .cuda_w4a16 import kernels as K

        self.ext = K.load_w4a16_extension()
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > K.MAX_RANKS:
            raise ValueError(f"at most {K.MAX_RANKS} ranks")
        self.max_n = (int(max_elems) + 7) // 8 * 8
        flag_bytes = 256 * ((self.SITES * self.world * 4 + 255) // 256)
        buf_bytes = 256 * ((self.SITES * self.world * self.max_n * 2 + 255) // 256)
        ll_bytes = self.SITES * self.world * self.max_n * 8      # {value, epoch} words of launches that push themselves
        self.mem = symm.empty(flag_bytes + buf_bytes + ll_bytes, dtype=torch.uint8, device=device)
        self.mem.zero_()
        self.handle = symm.rendezvous(self.mem, group)
        self.local = torch.zeros(64, dtype=torch.int32, device=device)   # [0:SITES] epochs, [32] status
        self.peers = K.Peers()
        ptrs = list(self.handle.buffer_ptrs)
        for r in range(self.world):
            self.peers.flag[r] = ptrs[r]
            self.peers.buf[r] = ptrs[r] + flag_bytes
            self.peers.ll_buf[r] = ptrs[r] + flag_bytes + buf_bytes
        self.peers.epoch = self.local.data_ptr()
        self.peers.status = self.local.data_ptr() + 32 * 4
        self.peers.world, self.peers.rank = self.world, self.rank
        self.peers.sites, self.peers.max_n = self.SITES, self.max_n
        self._calls = 0
        torch.cuda.synchronize(device)
        dist.barrier(group)          # every rank's flags are zero before anybody's first store arrives

    def all_reduce(self, t: torch.Tensor, site: int = None) -> torch.Tensor:
        """In-place sum of a contiguous fp16 tensor (numel % 8 == 0) on the current stream."""
        if t.dtype != torch.float16 or not t.is_contiguous() or t.numel() % 8:
            raise ValueError("expected a contiguous fp16 tensor with a multiple of 8 elements")
        if site is None:
            site = self._calls % self.SITES
            self._calls += 1
        rc = self.ext.lib.glowq_w4a16_allreduce_f16(self.peers, t.data_ptr(), t.numel(), int(site),
                                                    torch.cuda.current_stream(t.device).cuda_stream)
        self.ext.check(rc, "glowq_w4a16_allreduce_f16")
        return t

    def descriptor_address(self) -> int:
        """Address of the ``glowq_w4a16_peers_t`` (for ``Group.push``: the row-split launch stores its result into every
        rank's slot itself and its last CTAs write the sum over the ranks to the output)."""
        import ctypes
        return ctypes.addressof(self.peers)

    def finish(self, out: torch.Tensor, site: int) -> torch.Tensor:
        """Sum of the words a pushing launch on ``site`` left in this rank's buffer, written to ``out``.  The launch does
        this itself; the call remains for callers that want the sum in another buffer, and reproduces the same bits."""
        if out.dtype != torch.float16 or not out.is_contiguous() or out.numel() % 8:
            raise ValueError("expected a contiguous fp16 tensor with a multiple of 8 elements")
        rc = self.ext.lib.glowq_w4a16_allreduce_finish_f16(self.peers, out.data_ptr(), out.numel(), int(site),
                                                           torch.cuda.current_stream(out.device).cuda_stream)
        self.ext.check(rc, "glowq_w4a16_allreduce_finish_f16")
        return out

    def status(self) -> int:
        return int(self.local[32].item())
