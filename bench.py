#!/usr/bin/env python
"""Benchmark of the corrected W4A16 linears on a decoder-shaped stack (decode token steps).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--model llama-3.2-3b] [--impl reference]

One "step" is one decode token step of B tokens through every corrected linear of the stack (7 per layer, issued
as 4 fused group launches per layer).  Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement
of the reference path (oracle/) on the host cores instead; nothing else in this file executes oracle code except the
`cpu_baseline` leg of the default arm."""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# mean DRAM bytes (read + write) per gemv_stream_kernel launch of the Llama-3.2-3B batch-1 token step, from ncu
NCU_DRAM_BYTES_PER_LAUNCH = 14.38e6

# decode-sized vectors go through the one-CTA peer-store all-reduce; anything larger (prefill) through NCCL
PEER_AR_MAX_ELEMS = 64 * 1024

METRIC = "decode_tok_s"
UNIT = "tokens/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--model", default="llama-3.2-3b")
    ap.add_argument("--impl", default="glowq_b200", choices=["glowq_b200", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (debugging only)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--graph-collectives", action="store_true",
                    help="with N > 1, capture the NCCL all-reduces into the CUDA graph too (default: graphs per segment, "
                         "all-reduces launched between them)")
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="with N > 1: the library's peer-store all-reduce inside one CUDA graph per step (default), or "
                         "NCCL all-reduces between per-segment graphs")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--unfused", action="store_true", help="one launch per module (wrapper protocol) instead of per group")
    ap.add_argument("--split-k", type=int, default=0)
    ap.add_argument("--glowq-s-fraction", type=float, default=1.0,
                    help="GlowQ-S: fraction of the (layer, group) pairs that keep their correction (seed 3); the rest run "
                         "plain W4A16")
    ap.add_argument("--prefill-tokens", type=int, default=2048, help="tokens of the extra prefill (GEMM) measurement; 0 = skip")
    return ap.parse_args()


def workload_config(args, shape, extra=None):
    cfg = {"workload": f"{shape.name}-shaped stack, {args.layers or shape.layers} layers x 7 corrected W4A16 linears "
                       f"(g128, rank {shape.rank}), decode token step, batch {args.batch}",
           "scope": "linears only (the hot path); attention, norms, embedding and lm_head are not in the step",
           "batch": args.batch, "rank": shape.rank, "group_size": 128, "glowq_s_fraction": args.glowq_s_fraction,
           "l2_policy": "weights per step exceed L2 (inputs larger than L2)"}
    if extra:
        cfg.update(extra)
    return cfg


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu_index)],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:  # noqa: BLE001
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [v.strip() for v in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:  # noqa: BLE001
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# ------------------------------------------------------------------------------------------ reference arm (CPU)
def cpu_layer_inputs(shape, batch, n_distinct, seed=0):
    """Random packed weights / factors for `n_distinct` layers, as numpy arrays, without a quantiser pass
    (codes, zero-points and scales drawn directly with the value ranges RTN gives N(0, 0.02) weights)."""
    import numpy as np
    rng = np.random.default_rng(seed)
    s, r = shape, shape.rank
    layers = []

    def lin(oc, ic, bias=False):
        g = ic // 128
        return dict(qweight=rng.integers(-2**31, 2**31 - 1, size=(oc, ic // 8), dtype=np.int64).astype(np.int32),
                    qzeros=rng.integers(-2**31, 2**31 - 1, size=(oc, (g + 7) // 8), dtype=np.int64).astype(np.int32),
                    scales=(rng.uniform(0.006, 0.011, size=(oc, g))).astype(np.float16),
                    bias=(rng.standard_normal(oc) * 0.1).astype(np.float16) if bias else None,
                    L=(rng.standard_normal((oc, r)) * 0.01).astype(np.float16))

    def fac(ic):
        return (rng.standard_normal((r, ic)) * 0.01).astype(np.float16)

    for _ in range(n_distinct):
        layers.append([
            ("hidden", fac(s.hidden), [lin(s.q_out, s.hidden, s.qkv_bias), lin(s.kv_out, s.hidden, s.qkv_bias),
                                       lin(s.kv_out, s.hidden, s.qkv_bias)]),
            ("attn", fac(s.q_out), [lin(s.hidden, s.q_out)]),
            ("hidden", fac(s.hidden), [lin(s.inter, s.hidden), lin(s.inter, s.hidden)]),
            ("inter", fac(s.inter), [lin(s.hidden, s.inter)]),
        ])
    xs = {"hidden": rng.standard_normal((batch, s.hidden)).astype(np.float16),
          "attn": rng.standard_normal((batch, s.q_out)).astype(np.float16),
          "inter": rng.standard_normal((batch, s.inter)).astype(np.float16)}
    return layers, xs


def cpu_run_layer(C, layer, xs, threads):
    import numpy as np
    for inp, R, members in layer:
        x = xs[inp]
        r_io = np.zeros((x.shape[0], R.shape[0]), np.float32)
        for i, m in enumerate(members):   # the wrapper protocol: first member computes r, the others reuse it
            C.corrected_forward(x, m["qweight"], m["scales"], m["qzeros"], 128, bias=m["bias"], R=R, L=m["L"], alpha=1.0,
                                r_io=r_io, r_mode=1 if i == 0 else 2, num_threads=threads)


def run_reference(args, shape):
    """CPU restatement of the reference path on all host threads; one step = one full token step."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import c_oracle as C
    threads = os.cpu_count() or C.max_threads()
    n_layers = args.layers or shape.layers
    n_distinct = min(4, n_layers)
    layers, xs = cpu_layer_inputs(shape, args.batch, n_distinct)
    # bound the run: a full token step per timed step unless that would take minutes
    t0 = time.perf_counter()
    cpu_run_layer(C, layers[0], xs, threads)
    t_layer = time.perf_counter() - t0
    budget_s = 150.0
    layers_per_step = n_layers
    if t_layer * n_layers * (args.steps + args.warmup) > budget_s:
        layers_per_step = max(1, int(budget_s / (t_layer * (args.steps + args.warmup))))
    for w in range(args.warmup):
        for li in range(layers_per_step):
            cpu_run_layer(C, layers[li % n_distinct], xs, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for li in range(layers_per_step):
            cpu_run_layer(C, layers[li % n_distinct], xs, threads)
    dt = time.perf_counter() - t0
    ms_step = dt / args.steps * 1e3 * (n_layers / layers_per_step)
    value = args.batch / (ms_step / 1e3)
    sample = (f"{layers_per_step} of {n_layers} layers per timed step (scaled to the full stack), {n_distinct} distinct "
              f"random layers cycled, C restatement (oracle/w4a16_oracle.c) with OpenMP")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 accumulate over fp16 dequantised int4", "data": "synthetic",
            "config": workload_config(args, shape),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ GPU arm
def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback (6.65 TB/s, MEASURED_PEAKS.json absent)"


def run_gpu(args, shape):
    import torch
    import torch.distributed as dist
    from glowq_b200.cuda_w4a16 import kernels as K
    from glowq_b200.stack import LinearStack

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def log(msg):
        if args.verbose:
            print(f"[bench rank {rank}] {msg}", file=sys.stderr, flush=True)

    M = args.batch
    log("building the stack")
    enabled = None
    n_layers_cfg = args.layers or shape.layers
    if args.glowq_s_fraction < 1.0:
        # seeded subset of the 4 x layers (layer, group) pairs, as the selective-restoration sweep would enable them
        keys = []
        for li in range(n_layers_cfg):
            keys += [f"layer{li}_qkv", f"model.layers.{li}.self_attn.o_proj", f"layer{li}_mlp",
                     f"model.layers.{li}.mlp.down_proj"]
        gsel = torch.Generator().manual_seed(3)
        perm = torch.randperm(len(keys), generator=gsel)[:int(round(args.glowq_s_fraction * len(keys)))]
        enabled = {keys[i] for i in perm.tolist()}
    stack = LinearStack(shape, dev, seed=0, layers=args.layers, tp_rank=rank, tp_world=world, enabled_groups=enabled)
    log("stack built")
    stream = torch.cuda.Stream(dev)
    with torch.cuda.stream(stream):
        plan = stack.plan(M, corrected=True, fuse_groups=not args.unfused, split_k=args.split_k)
        plain = stack.plan(M, corrected=False, fuse_groups=not args.unfused, split_k=args.split_k)
    n_layers = len(stack.groups) // 4
    calls_per_layer = plan["n"] // n_layers

    # outputs that a row-split linear must sum across ranks (o_proj, down_proj): the natural all-reduce points
    def reduce_points(p):
        pts = []
        idx = 0
        for g in stack.groups:
            n = 1 if not args.unfused else len(g.members)
            idx += n
            if g.input_name in ("attn", "inter"):
                pts.append(idx)
        return pts

    peer_ar = None
    if world > 1 and args.collective == "peer":
        try:
            from glowq_b200.tp import PeerAllReduce
            peer_ar = PeerAllReduce(dist.group.WORLD, dev, max_elems=PEER_AR_MAX_ELEMS)
            log("peer all-reduce ready")
        except Exception as exc:  # noqa: BLE001 - symmetric memory unavailable: fall back to NCCL
            print(f"[bench] peer all-reduce unavailable ({exc!r}); using NCCL", file=sys.stderr, flush=True)
            peer_ar = None

    def make_step(p):
        """(callable that enqueues one step, list of segments).  With one rank a step is one C call; with N ranks it is
        a list of (group calls, tensor to all-reduce) segments ending at the row-split linears."""
        if world == 1:
            return (lambda: stack.step(p)), None
        pts = reduce_points(p)
        ptr2t = {}
        for item in p["keep"]:
            if isinstance(item, list):
                for t in item:
                    ptr2t[t.data_ptr()] = t
        segs = []
        start = 0
        for e in pts:
            arr = (K.Group * (e - start))(*[p["calls"][i] for i in range(start, e)])
            segs.append((arr, e - start, ptr2t[p["calls"][e - 1].members[0].out]))
            start = e

        if peer_ar is not None and all(t.numel() <= PEER_AR_MAX_ELEMS for _, _, t in segs):
            def step():
                for i, (arr, n, t) in enumerate(segs):
                    stack.ext.check(stack.ext.lib.glowq_w4a16_group_forward_many(arr, n), "group_forward_many")
                    peer_ar.all_reduce(t, site=i & 1)
            return step, None          # plain kernels only: the whole step goes into one CUDA graph

        def step():
            for arr, n, t in segs:
                stack.ext.check(stack.ext.lib.glowq_w4a16_group_forward_many(arr, n), "group_forward_many")
                dist.all_reduce(t)
        return step, segs

    def timed(step_and_segs, steps, warmup, use_graph):
        step_fn, segs = step_and_segs
        with torch.cuda.stream(stream):
            for _ in range(max(3, warmup)):
                step_fn()
            stream.synchronize()
            run = step_fn
            if use_graph and (segs is None or args.graph_collectives):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    step_fn()
                run = graph.replay
            elif use_graph:
                # one graph per segment of group launches; the all-reduces are enqueued between the replays
                graphs = []
                for arr, n, t in segs:
                    g_ = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g_, stream=stream):
                        stack.ext.check(stack.ext.lib.glowq_w4a16_group_forward_many(arr, n), "group_forward_many")
                    graphs.append((g_, t))

                def run():
                    for g_, t in graphs:
                        g_.replay()
                        dist.all_reduce(t)
            for _ in range(3):
                run()
            stream.synchronize()
            log("warm-up done")
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                run()
            e1.record(stream)
            stream.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            if world > 1:
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            log(f"timed {steps} steps: {ms / steps:.4f} ms/step")
        return ms / steps, run

    use_graph = not args.no_graph
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_step, run = timed(make_step(plan), args.steps, args.warmup, use_graph)
    clocks = sampler.stop() if rank == 0 else {}
    ms_plain, _ = timed(make_step(plain), args.steps, args.warmup, use_graph)
    stack.check_status(plan)

    # end to end: host activations in, result out, every step
    with torch.cuda.stream(stream):
        host_in = {k: v.cpu().pin_memory() for k, v in plan["inputs"].items()}
        last = plan["last_out"]
        host_out = torch.empty_like(last, device="cpu").pin_memory()
        for _ in range(3):
            for k, v in plan["inputs"].items():
                v.copy_(host_in[k], non_blocking=True)
            run()
            host_out.copy_(last, non_blocking=True)
            stream.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        e2e_steps = min(args.steps, 200)
        for _ in range(e2e_steps):
            for k, v in plan["inputs"].items():
                v.copy_(host_in[k], non_blocking=True)
            run()
            host_out.copy_(last, non_blocking=True)
            stream.synchronize()
        e2e_ms = (time.perf_counter() - t0) / e2e_steps * 1e3
        if world > 1:
            t = torch.tensor([e2e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
    h2d = sum(v.numel() * v.element_size() for v in plan["inputs"].values())
    d2h = last.numel() * last.element_size()

    # extra: prefill pass of the same stack through the tensor-core GEMM (reported, not the headline value)
    prefill = None
    if args.prefill_tokens > 0:
        Mp = args.prefill_tokens
        with torch.cuda.stream(stream):
            pplan = stack.plan(Mp, corrected=True, fuse_groups=not args.unfused)
        ms_p, _ = timed(make_step(pplan), max(3, min(10, args.steps)), 3, False)
        stack.check_status(pplan)
        fl = stack.algorithmic_flops(Mp, corrected=True)
        prefill = {"tokens": Mp, "ms": ms_p, "tokens_per_s": Mp / (ms_p * 1e-3), "tflops": fl / (ms_p * 1e-3) / 1e12,
                   "kernel": "gemm_w4a16_kernel (tcgen05)", "flops_per_pass": fl}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peaks()
    if prefill is not None:
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                mp_ = json.load(f)
            prefill["frac_of_measured_bf16_burst"] = prefill["tflops"] * world / float(mp_["bf16_tflops"]) / world
            prefill["frac_of_measured_bf16_sustained"] = prefill["tflops"] / float(mp_["bf16_tflops_sustained"])
        except Exception:  # noqa: BLE001
            pass
        prefill["frac_of_nominal_fp16_dense"] = prefill["tflops"] / 2250.0
    alg = stack.algorithmic_bytes(M, corrected=True)
    alg_plain = stack.algorithmic_bytes(M, corrected=False)
    achieved = alg / (ms_step * 1e-3) / 1e9
    line = {"metric": METRIC, "value": M / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 accumulate over fp16 x int4 (tensor-core MMA), fp16 out",
            "data": "synthetic",
            "config": workload_config(args, shape, {"parallelism": f"tp{world}", "cuda_graph": use_graph,
                                                    "collective": ("peer-store all-reduce kernel" if peer_ar is not None
                                                                   else "nccl") if world > 1 else None,
                                                    "launches_per_layer": calls_per_layer}),
            "clocks": {k: clocks.get(k) for k in ("sm_mhz", "sm_max_mhz", "reasons")},
            "e2e": {"value": M / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms},
            "gpu_launches": plan["n"] * args.steps,
            "roofline": {"bound": "hbm", "kernel": "gemv_stream_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "frac_of_8tbs": achieved / 8000.0,
                         "traffic": NCU_DRAM_BYTES_PER_LAUNCH if shape.name == "llama-3.2-3b" and M == 1 and world == 1 else None,
                         "traffic_source": "profiles/gemv_stream_llama32_3b_decode_launches.md (ncu dram__bytes_read+write, "
                                           "mean over the launches of a token step)",
                         "peak_source": peak_src, "bytes_per_launch": alg / plan["n"],
                         "us_per_launch": ms_step * 1e3 / plan["n"], "launches_per_step": plan["n"],
                         "note": "algorithmic bytes of one launch (mean over the step's launches) / mean launch duration "
                                 "from CUDA events around the graph-replayed step (inter-kernel gaps included)"},
            "correction_overhead": {"time_ratio": ms_step / ms_plain, "plain_ms_per_step": ms_plain,
                                    "byte_ratio_floor": alg / alg_plain},
            "prefill": prefill}
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = gpu_arm_cpu_baseline(args, shape)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def gpu_arm_cpu_baseline(args, shape):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import c_oracle as C
    threads = os.cpu_count() or C.max_threads()
    layers, xs = cpu_layer_inputs(shape, args.batch, 1)
    cpu_run_layer(C, layers[0], xs, threads)
    reps, t0 = 0, time.perf_counter()
    while reps < 3 or (time.perf_counter() - t0 < 10.0 and reps < 200):
        cpu_run_layer(C, layers[0], xs, threads)
        reps += 1
    t_layer = (time.perf_counter() - t0) / reps
    n_layers = args.layers or shape.layers
    return {"value": args.batch / (t_layer * n_layers), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"1 of {n_layers} layers x {reps} repetitions (~10 s), scaled by the layer count; "
                      f"C restatement of the reference CPU path with OpenMP"}


def main():
    args = parse_args()
    from glowq_b200.stack import SHAPES
    shape = SHAPES[args.model]
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return
        run_reference(args, shape)
        return
    run_gpu(args, shape)


if __name__ == "__main__":
    main()
