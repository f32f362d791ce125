"""The peer-store all-reduce against NCCL on two GPUs (skipped on a single-GPU box)."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist
    from glowq_b200.tp import PeerAllReduce
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        ar = PeerAllReduce(dist.group.WORLD, dev, max_elems=4 * 3072)
        gen = torch.Generator(device=dev).manual_seed(100 + rank)
        worst = 0.0
        for it in range(40):
            n = (3072, 8 * 3072 // 8, 4 * 3072, 8)[it % 4]
            x = torch.randn(n, generator=gen, device=dev).half()
            want = x.float().clone()
            dist.all_reduce(want)
            got = ar.all_reduce(x.clone())
            torch.cuda.synchronize()
            worst = max(worst, float((got.float() - want).abs().max()))
        # replay from a CUDA graph: the collective is an ordinary kernel.  The graph holds two calls on alternating
        # sites (a site may only be reused once every rank has finished its previous call on it, which the call on the
        # other site in between guarantees), and the data change between replays.
        xa = torch.zeros(3072, dtype=torch.float16, device=dev)
        xb = torch.zeros(4 * 3072, dtype=torch.float16, device=dev)
        s = torch.cuda.Stream(dev)
        with torch.cuda.stream(s):
            ar.all_reduce(xa, site=0)
            ar.all_reduce(xb, site=1)
            s.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                ar.all_reduce(xa, site=0)
                ar.all_reduce(xb, site=1)
            s.synchronize()
            for rep in range(4):
                va = torch.randn(3072, generator=gen, device=dev).half()
                vb = torch.randn(4 * 3072, generator=gen, device=dev).half()
                wa, wb = va.float().clone(), vb.float().clone()
                s.synchronize()
                dist.all_reduce(wa)
                dist.all_reduce(wb)
                torch.cuda.synchronize()
                xa.copy_(va)
                xb.copy_(vb)
                g.replay()
                s.synchronize()
                worst = max(worst, float((xa.float() - wa).abs().max()), float((xb.float() - wb).abs().max()))
        q.put((rank, worst, ar.status()))
    finally:
        dist.destroy_process_group()


def test_peer_allreduce_matches_nccl():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, worst, status in res:
        assert status == 0, (rank, status)
        assert worst <= 2e-2, (rank, worst)       # fp16 rounding of a sum of two O(1) values


_EXPIRY_SCRIPT = r"""
import ctypes, sys, torch
from glowq_b200.cuda_w4a16 import kernels as K
ext = K.load_w4a16_extension()
dev = torch.device("cuda", 0)
world, sites, max_n = 2, 2, 1024
mem = [torch.zeros(sites * world * max_n, dtype=torch.float16, device=dev) for _ in range(world)]
flags = [torch.zeros(sites * world, dtype=torch.int32, device=dev) for _ in range(world)]
local = torch.zeros(64, dtype=torch.int32, device=dev)
p = K.Peers()
for r in range(world):                       # "rank 1" is local memory that nobody ever writes flags into
    p.buf[r], p.flag[r] = mem[r].data_ptr(), flags[r].data_ptr()
p.epoch, p.status = local.data_ptr(), local.data_ptr() + 32 * 4
p.world, p.rank, p.sites, p.max_n = world, 0, sites, max_n
x = torch.ones(1024, dtype=torch.float16, device=dev)
rc = ext.lib.glowq_w4a16_allreduce_f16(p, x.data_ptr(), 1024, 0, torch.cuda.current_stream().cuda_stream)
torch.cuda.synchronize()                     # the kernel returned although rank 1 never arrived
print("RC", rc, "STATUS", int(local[32].item()), "FLAG0", int(flags[0][0].item()), "FLAG1", int(flags[1][0].item()))
"""


def test_bounded_wait_runs_out_when_a_rank_never_arrives():
    """One GPU: a two-rank descriptor whose second rank is plain local memory that nobody launches for.  With the poll
    limit set short (read once per process, hence the child interpreter) the kernel gives up, records status 4 and
    returns; the context stays usable."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, GLOWQ_AR_SPIN_LIMIT="2000", PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-c", _EXPIRY_SCRIPT], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "RC 0 STATUS 4 FLAG0 1 FLAG1 1" in r.stdout, r.stdout[-2000:]
