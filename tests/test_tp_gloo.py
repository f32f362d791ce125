"""Tensor-parallel sharding on CPU ranks (gloo, world size 2 and 3): shard, compute each shard with the CPU oracle,
combine with the collective the layout prescribes, compare with the unsharded oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import glowq_oracle as O
from glowq_b200 import CudaW4A16Linear
from glowq_b200 import tp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_forward(mod, x, R=None, L=None, alpha=1.0):
    deq = O.dequant_full(mod.qweight_i32.numpy(), mod.qzeros_i32.numpy(), mod.scales_f16.numpy(), mod.in_features,
                         mod.group_size)
    bias = None if mod.bias is None else mod.bias.data.numpy()
    return O.corrected_forward_fp32(x, deq, None if R is None else R.numpy(), None if L is None else L.numpy(), alpha, bias)


def _make(seed, oc, ic, rank, bias):
    g = torch.Generator().manual_seed(seed)
    lin = torch.nn.Linear(ic, oc, bias=bias).half()
    lin.weight.data.copy_((torch.randn(oc, ic, generator=g) * 0.02).half())
    if bias:
        lin.bias.data.copy_((torch.randn(oc, generator=g) * 0.1).half())
    mod = CudaW4A16Linear.from_float(lin, 128)
    R = (torch.randn(rank, ic, generator=g) * 0.01).half()
    L = (torch.randn(oc, rank, generator=g) * 0.01).half()
    x = torch.randn(3, ic, generator=g).half().numpy()
    return mod, R, L, x


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # column-parallel: rows split, R replicated, outputs gathered
        mod, R, L, x = _make(0, 256, 384, 16, True)
        want = _oracle_forward(mod, x, R, L, 0.5)
        sh, L_sh = tp.column_parallel_shard(mod, rank, world, multiple=128 if world == 2 else 1, L=L)
        y = torch.from_numpy(_oracle_forward(sh, x, R, L_sh, 0.5))
        sizes = [b - a for a, b in tp.row_bounds(256, world, 128 if world == 2 else 1)]
        parts = [torch.empty(3, s) for s in sizes]
        if len(set(sizes)) == 1:
            dist.all_gather(parts, y)
        else:
            for r in range(world):
                parts[r] = y.clone() if r == rank else parts[r]
                dist.broadcast(parts[r], src=r)
        got = torch.cat(parts, dim=1).numpy()
        err_col = float(np.abs(got - want).max())

        # row-parallel: 5 groups over `world` ranks (uneven), zero words re-packed, all-reduce
        mod, R, L, x = _make(1, 96, 640, 16, True)
        want = _oracle_forward(mod, x, R, L, 1.0)
        sh, R_sh, (c0, c1) = tp.row_parallel_shard(mod, rank, world, R=R)
        y = torch.from_numpy(_oracle_forward(sh, x[:, c0:c1], R_sh, L, 1.0))
        dist.all_reduce(y)
        err_row = float(np.abs(y.numpy() - want).max())
        q.put((rank, err_col, err_row, (c0, c1)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_tp_shards_reproduce_the_unsharded_linear(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err_col, err_row, _ in results:
        assert err_col <= 1e-5, (rank, err_col)
        assert err_row <= 1e-4, (rank, err_row)
    cols = sorted(c for *_, c in results)
    assert cols[0][0] == 0 and cols[-1][1] == 640 and all(a[1] == b[0] for a, b in zip(cols, cols[1:]))


def test_group_bounds_llama2_13b_down_proj_over_8():
    b = tp.group_bounds(13824 // 128, 8)
    assert [e - s for s, e in b] == [14, 14, 14, 14, 13, 13, 13, 13]
    assert tp.row_bounds(13824, 8, 128)[0] == (0, 1792) and tp.row_bounds(13824, 8, 128)[-1] == (12160, 13824)
    with pytest.raises(ValueError):
        tp.row_bounds(100, 2, 128)
