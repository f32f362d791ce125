"""Single-launch micro-benchmark of the corrected W4A16 kernels on named shapes.

    python microbench.py --shapes gu14b,qkv3b --M 1,8 --modes plain,corr [--kernel 0|1|2] [--iters N]

Every configuration is timed as a CUDA-graph replay over enough distinct weight copies to exceed L2, with CUDA events
on the launching stream; one JSON line per (shape, M, mode) with microseconds per launch, algorithmic GB/s (and its
fraction of the measured copy bandwidth) and TFLOP/s.  Modes: plain (no correction), corr (this launch computes
r = R x), load (r is read from the group's buffer)."""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from glowq_b200.cuda_w4a16 import kernels as K  # noqa: E402
from glowq_b200.stack import QLinear  # noqa: E402

SHAPES = {  # name: (output rows of each member, input columns, rank)
    "qkv3b": ([3072, 1024, 1024], 3072, 64), "o3b": ([3072], 3072, 64), "gu3b": ([8192, 8192], 3072, 64),
    "down3b": ([3072], 8192, 64), "k3b": ([1024], 3072, 64),
    "qkv7b": ([3584, 512, 512], 3584, 128), "gu7b": ([18944, 18944], 3584, 128), "down7b": ([3584], 18944, 128),
    "qkv13b": ([5120, 5120, 5120], 5120, 128), "gu13b": ([13824, 13824], 5120, 128), "down13b": ([5120], 13824, 128),
    "o13b": ([5120], 5120, 128),
    "qkv14b": ([5120, 1024, 1024], 5120, 256), "o14b": ([5120], 5120, 256), "gu14b": ([17408, 17408], 5120, 256),
    "down14b": ([5120], 17408, 256), "opt_qkv": ([2048, 2048, 2048], 2048, 64),
    # one rank's shards of the Llama-2-13B layer under 2- and 8-way tensor parallelism
    "qkv13b_tp2": ([2560, 2560, 2560], 5120, 128), "o13b_tp2": ([5120], 2560, 128),
    "gu13b_tp2": ([6912, 6912], 5120, 128), "down13b_tp2": ([5120], 6912, 128),
    "qkv13b_tp8": ([640, 640, 640], 5120, 128), "o13b_tp8": ([5120], 640, 128),
    "gu13b_tp8": ([1728, 1728], 5120, 128), "down13b_tp8": ([5120], 1792, 128),
}


def measured_hbm_gbs() -> float:
    try:
        root = os.path.dirname(os.path.abspath(__file__))
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"])
    except Exception:  # noqa: BLE001
        return 6650.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="qkv3b,o3b,gu3b,down3b")
    ap.add_argument("--M", default="1")
    ap.add_argument("--modes", default="plain,corr")
    ap.add_argument("--split-k", type=int, default=0)
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--no-chain", action="store_true", help="leave the `next` hint of every call empty")
    ap.add_argument("--kernel", type=int, default=0, help="0 auto, 1 weight-streaming kernel, 2 tensor-core GEMM")
    args = ap.parse_args()
    ext = K.load_w4a16_extension()
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(0)
    peak = measured_hbm_gbs()
    for name in args.shapes.split(","):
        ocs, ic, rank = SHAPES[name]
        wbytes = sum(oc * ic // 2 for oc in ocs)
        ncopies = max(2, min(64, (300 << 20) // wbytes + 1))
        copies = []
        for _ in range(ncopies):
            lins = [QLinear(oc, ic, rank, gen, dev) for oc in ocs]
            R = (torch.randn(rank, ic, generator=gen, device=dev) * 0.01).half()
            copies.append((lins, R))
        for M in [int(m) for m in args.M.split(",")]:
            x = torch.randn(M, ic, generator=gen, device=dev).half()
            for mode in args.modes.split(","):
                st = torch.cuda.Stream()
                groups, keep = [], []
                for lins, R in copies:
                    g = K.Group()
                    g.x, g.M, g.IC, g.x_stride = x.data_ptr(), M, ic, ic
                    g.group_size, g.kernel, g.split_k = 128, args.kernel, args.split_k
                    r_buf = torch.zeros(M, rank, dtype=torch.float16, device=dev)
                    if mode == "corr":
                        g.rank, g.r_mode, g.R, g.R_stride, g.r_buf = rank, K.R_COMPUTE, R.data_ptr(), ic, r_buf.data_ptr()
                    elif mode == "load":
                        g.rank, g.r_mode, g.r_buf = rank, K.R_LOAD, r_buf.data_ptr()
                    g.n_members = len(lins)
                    outs = []
                    for i, l in enumerate(lins):
                        o = torch.empty(M, l.oc, dtype=torch.float16, device=dev)
                        outs.append(o)
                        m = g.members[i]
                        m.qweight, m.scales, m.qzeros = l.qweight.data_ptr(), l.scales.data_ptr(), l.qzeros.data_ptr()
                        if mode != "plain":
                            m.L, m.L_stride = l.L.data_ptr(), rank
                        m.out, m.out_stride, m.OC = o.data_ptr(), l.oc, l.oc
                        m.weight_stride_i32, m.zero_stride_i32 = l.qweight.stride(0), l.qzeros.stride(0)
                        m.scale_stride, m.alpha = l.scales.stride(0), 1.0
                    ws = ext.new_workspace(ext.workspace_bytes(M, ic, sum(ocs), rank, len(lins)) + (64 << 20), dev)
                    g.workspace, g.workspace_bytes, g.stream = ws.data_ptr(), ws.numel(), st.cuda_stream
                    groups.append(g)
                    keep += [outs, ws, r_buf]
                arr = (K.Group * len(groups))(*groups)
                n = len(groups)
                if not args.no_chain:   # every launch names the one that follows it on the stream
                    for i in range(n):
                        arr[i].next = ctypes.addressof(arr[(i + 1) % n])
                with torch.cuda.stream(st):
                    for _ in range(2):
                        ext.check(ext.lib.glowq_w4a16_group_forward_many(arr, n))
                    st.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=st):
                        ext.lib.glowq_w4a16_group_forward_many(arr, n)
                    graph.replay()
                    st.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    reps = max(1, args.iters // n)
                    e0.record(st)
                    for _ in range(reps):
                        graph.replay()
                    e1.record(st)
                    st.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / (reps * n)
                G = ic // 128
                b = sum(oc * ic // 2 + oc * G * 2 + oc * ((G + 7) // 8) * 4 + M * oc * 2 for oc in ocs) + M * ic * 2
                if mode != "plain":
                    b += sum(oc * rank * 2 for oc in ocs)
                if mode == "corr":
                    b += rank * ic * 2
                flops = 2.0 * M * sum(ocs) * ic
                if mode != "plain":
                    flops += 2.0 * M * sum(ocs) * rank
                if mode == "corr":
                    flops += 2.0 * M * rank * ic
                status = ext.lib.glowq_w4a16_read_status(groups[0].workspace, groups[0].stream)
                print(json.dumps({"shape": name, "M": M, "mode": mode, "us": round(us, 2), "GBs": round(b / us / 1e3, 1),
                                  "frac_of_measured_hbm": round(b / us / 1e3 / peak, 3), "TFs": round(flops / us / 1e6, 1),
                                  "status": status, "copies": n}), flush=True)
        del copies


if __name__ == "__main__":
    main()
