#!/usr/bin/env python
"""Benchmark of the corrected W4A16 linears on a decoder-shaped stack (decode token steps).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--model llama-2-13b] [--impl reference]

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
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# mean DRAM bytes (read + write) per gemv_stream_kernel launch of a batch-1 token step, from ncu captures of this
# bench command (profiles/gemv_stream_*_decode_launches.md), keyed by (model, batch)
NCU_DRAM_BYTES_PER_LAUNCH = {("llama-3.2-3b", 1): 14.38e6, ("llama-2-13b", 1): 46.58e6}

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
    ap.add_argument("--model", default="llama-2-13b")
    ap.add_argument("--impl", default="glowq_b200", choices=["glowq_b200", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (debugging only)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="with N > 1: the library's peer-store all-reduce inside one CUDA graph per step (default), or "
                         "NCCL all-reduces between per-segment graphs")
    ap.add_argument("--push", default="auto", choices=["auto", "on", "off"],
                    help="with N > 1: let the row-split linears store their partial sums to the peers from their own "
                         "epilogue and complete the sum in their last CTAs (group.push) instead of the one-launch peer "
                         "all-reduce that follows them. auto: wherever the launch can (up to 8 tokens)")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="skip the extra `sweep` and `e2e_host_entry` measurements")
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


def glowq_s_mask(n_layers, fraction):
    """Seeded subset (seed 3) of the 4 x layers (layer, group) pairs that keep their correction, as the
    selective-restoration sweep would enable them; None = all."""
    import torch
    if fraction >= 1.0:
        return None
    keys = []
    for li in range(n_layers):
        keys += [f"layer{li}_qkv", f"model.layers.{li}.self_attn.o_proj", f"layer{li}_mlp",
                 f"model.layers.{li}.mlp.down_proj"]
    gsel = torch.Generator().manual_seed(3)
    perm = torch.randperm(len(keys), generator=gsel)[:int(round(fraction * len(keys)))]
    return {keys[i] for i in perm.tolist()}


class GpuArm:
    """One process of the GPU arm: device, (optional) process group, timing helpers."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.args = torch, dist, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and self.world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=self.dev)
        self.stream = torch.cuda.Stream(self.dev)
        self.peer_ar = None
        if self.world > 1 and args.collective == "peer":
            try:
                from glowq_b200.tp import PeerAllReduce
                self.peer_ar = PeerAllReduce(dist.group.WORLD, self.dev, max_elems=PEER_AR_MAX_ELEMS)
            except Exception as exc:  # noqa: BLE001 - symmetric memory unavailable: NCCL between graph segments
                print(f"[bench] peer all-reduce unavailable ({exc!r}); using NCCL", file=sys.stderr, flush=True)

    def log(self, msg):
        if self.args.verbose:
            print(f"[bench rank {self.rank}] {msg}", file=sys.stderr, flush=True)

    def build_stack(self, shape, layers=None, fraction=1.0):
        from glowq_b200.stack import LinearStack
        n_layers = layers or shape.layers
        return LinearStack(shape, self.dev, seed=0, layers=layers, tp_rank=self.rank, tp_world=self.world,
                           enabled_groups=glowq_s_mask(n_layers, fraction))

    # -------------------------------------------------------------------------------------- one step
    def make_step(self, stack, p):
        """(callable that enqueues one step, segments or None).  One rank: a step is one C call.  N ranks: the group
        calls up to each row-split linear (o_proj, down_proj), then the all-reduce of its output - the library's
        peer-store kernel (whole step capturable in one CUDA graph), or NCCL between per-segment graphs."""
        from glowq_b200.cuda_w4a16 import kernels as K
        dist = self.dist
        if self.world == 1:
            return (lambda: stack.step(p)), None
        segs, start, idx = [], 0, 0
        for g, outs in zip(stack.groups, p["group_outs"]):
            idx += len(g.members) if self.args.unfused else 1
            if g.input_name in ("attn", "inter"):
                arr = (K.Group * (idx - start))(*[p["calls"][i] for i in range(start, idx)])
                segs.append((arr, idx - start, outs[0]))
                start = idx
        lib, check = stack.ext.lib, stack.ext.check
        if self.peer_ar is not None and all(t.numel() <= PEER_AR_MAX_ELEMS for _, _, t in segs):
            pushed = all(arr[n - 1].push for arr, n, _ in segs)    # the row-split launches store to the peers themselves

            def step():
                for i, (arr, n, t) in enumerate(segs):
                    check(lib.glowq_w4a16_group_forward_many(arr, n), "group_forward_many")
                    if not pushed:   # a pushing launch completes the sum itself
                        self.peer_ar.all_reduce(t, site=i & 1)
            return step, None

        def step():
            for arr, n, t in segs:
                check(lib.glowq_w4a16_group_forward_many(arr, n), "group_forward_many")
                dist.all_reduce(t)
        return step, segs

    def timed(self, stack, step_and_segs, steps, warmup, use_graph):
        """ms per step (CUDA events on the launching stream, max over ranks) and the callable that runs one step."""
        torch, dist, stream = self.torch, self.dist, self.stream
        step_fn, segs = step_and_segs
        if self.world > 1:
            dist.barrier()       # the ranks enter their first step together (the in-kernel waits for a peer are bounded)
        with torch.cuda.stream(stream):
            for _ in range(max(3, warmup)):
                step_fn()
            stream.synchronize()
            run = step_fn
            if use_graph and segs is None:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    step_fn()
                run = graph.replay
            elif use_graph:
                # one graph per segment of group launches; the NCCL all-reduces are enqueued between the replays
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
            if self.world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                run()
            e1.record(stream)
            stream.synchronize()
            if self.world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            if self.world > 1:
                t = torch.tensor([ms], device=self.dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
        return ms / steps, run

    def pushes(self, M):
        """Whether the row-split launches of an M-token step store to the peers themselves."""
        if self.world == 1 or self.peer_ar is None or self.args.push == "off":
            return False
        return M <= 8   # the weight-streaming kernel's launches; larger batches take the GEMM and the separate all-reduce

    def decode(self, stack, M, steps, warmup, corrected=True):
        """Time one decode configuration; returns (ms per step, run callable, plan)."""
        torch = self.torch
        with torch.cuda.stream(self.stream):
            plan = stack.plan(M, corrected=corrected, fuse_groups=not self.args.unfused, split_k=self.args.split_k,
                              push=self.peer_ar if self.pushes(M) else None)
        ms, run = self.timed(stack, self.make_step(stack, plan), steps, warmup, not self.args.no_graph)
        stack.check_status(plan)
        return ms, run, plan

    # -------------------------------------------------------------------------------------- tensor-parallel parity
    def tp_parity(self, stack, plan):
        """N > 1: run one eager step with its all-reduces and compare layer 0's o_proj and down_proj outputs (the sums
        over the ranks' partial results) with the CPU oracle of the UNSHARDED linears on the full activations."""
        torch, dist = self.torch, self.dist
        step_fn, _ = self.make_step(stack, plan)
        with torch.cuda.stream(self.stream):
            step_fn()
            self.stream.synchronize()
        dist.barrier()
        out = None
        if self.rank == 0:
            sys.path.insert(0, os.path.join(ROOT, "oracle"))
            import numpy as np
            import c_oracle as C
            worst_abs = worst_rel = 0.0
            for gi, key, inp in ((1, "o_proj", "attn"), (3, "down_proj", "inter")):
                ref = stack.tp_reference[key]
                x = plan["full_inputs"][inp].cpu().numpy()
                want = C.corrected_forward(x, ref["qweight"], ref["scales"], ref["qzeros"], 128, bias=ref["bias"],
                                           R=ref["R"], L=ref["L"], alpha=1.0)
                got = plan["group_outs"][gi][0].float().cpu().numpy()
                worst_abs = max(worst_abs, float(np.abs(got - want).max()))
                worst_rel = max(worst_rel, float(np.abs(got - want).mean() / np.abs(want).mean()))
            out = {"max_abs": worst_abs, "mean_rel": worst_rel, "tolerance": {"max_abs": 2e-2, "mean_rel": 1e-3},
                   "checked": "layer 0 o_proj and down_proj, all-reduced over the ranks, against the C oracle of the "
                              "unsharded linears", "ok": worst_abs <= 2e-2 and worst_rel <= 1e-3}
        dist.barrier()
        return out


def run_gpu(args, shape):
    arm = GpuArm(args)
    torch, dist, world, rank = arm.torch, arm.dist, arm.world, arm.rank
    M = args.batch
    use_graph = not args.no_graph
    arm.log("building the stack")
    stack = arm.build_stack(shape, args.layers, args.glowq_s_fraction)
    arm.log("stack built")
    n_layers = len(stack.groups) // 4

    sampler = ClockSampler(arm.local)
    if rank == 0:
        sampler.start()
    ms_step, run, plan = arm.decode(stack, M, args.steps, args.warmup, corrected=True)
    clocks = sampler.stop() if rank == 0 else {}
    ms_plain, _, _ = arm.decode(stack, M, args.steps, args.warmup, corrected=False)
    calls_per_layer = plan["n"] // n_layers
    tp_par = arm.tp_parity(stack, plan) if world > 1 else None

    # end to end: activations come from pinned host memory every step and the last output goes back, around the same
    # graph-replayed step (torch copies on the launching stream, one synchronisation per step)
    stream = arm.stream
    with torch.cuda.stream(stream):
        host_in = {k: v.cpu().pin_memory() for k, v in plan["inputs"].items()}
        last = plan["last_out"]
        host_out = torch.empty_like(last, device="cpu").pin_memory()

        def e2e_step():
            for k, v in plan["inputs"].items():
                v.copy_(host_in[k], non_blocking=True)
            run()
            host_out.copy_(last, non_blocking=True)
            stream.synchronize()
        for _ in range(3):
            e2e_step()
        if world > 1:
            dist.barrier()
        e2e_steps = min(args.steps, 200)
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        e2e_ms = (time.perf_counter() - t0) / e2e_steps * 1e3
        if world > 1:
            t = torch.tensor([e2e_ms], device=arm.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
    h2d = sum(v.numel() * v.element_size() for v in plan["inputs"].values())
    d2h = last.numel() * last.element_size()

    # the same step with every group call going through the C ABI's host-buffer entry point (copy in, launch, copy out,
    # synchronise - per group): what a caller without device-resident activations pays
    host_entry = dropin = None
    if world == 1 and not args.no_sweep:
        host_entry = host_entry_step(arm, stack, plan, min(args.steps, 20))
        dropin = dropin_step(arm, stack, plan, min(args.steps, 50))

    # extra: prefill pass of the same stack through the tensor-core GEMM (reported, not the headline value)
    prefill = None
    if args.prefill_tokens > 0:
        prefill = measure_prefill(arm, stack, args.prefill_tokens, max(3, min(10, args.steps)))

    alg = stack.algorithmic_bytes(M, corrected=True)
    alg_plain = stack.algorithmic_bytes(M, corrected=False)
    del plan, run
    stack._plans.clear()
    torch.cuda.empty_cache()

    sweep = None
    if world == 1 and not args.no_sweep:
        sweep = run_sweep(arm, args, stack if (args.layers is None and args.glowq_s_fraction >= 1.0) else None)
    del stack

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peaks()
    achieved = alg / (ms_step * 1e-3) / 1e9
    n_calls = calls_per_layer * n_layers
    traffic = NCU_DRAM_BYTES_PER_LAUNCH.get((shape.name, M)) if world == 1 and args.glowq_s_fraction >= 1.0 else None
    line = {"metric": METRIC, "value": M / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 accumulate over fp16 x int4 (tensor-core MMA), fp16 out",
            "data": "synthetic", "config": workload_config(args, shape),
            "plan": {"parallelism": f"tp{world}", "cuda_graph": use_graph,
                     "collective": ((("inside the row-split launch (peer stores from its epilogue, summed by its last CTAs)" if arm.pushes(M)
                                      else "peer-store all-reduce kernel") if arm.peer_ar is not None else "nccl")
                                    if world > 1 else None),
                     "launches_per_layer": calls_per_layer},
            "clocks": {k: clocks.get(k) for k in ("sm_mhz", "sm_max_mhz", "reasons")},
            "e2e": {"value": M / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms,
                    "path": "pinned-host activations copied in and the last output copied out every step (torch "
                            "copy_ on the launching stream) around the graph-replayed step; see e2e_host_entry for the "
                            "C ABI's own host-buffer call"},
            "e2e_host_entry": host_entry, "dropin": dropin,
            "gpu_launches": n_calls * args.steps,
            "roofline": {"bound": "hbm", "kernel": "gemv_stream_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "frac_of_8tbs": achieved / 8000.0,
                         "traffic": traffic,
                         "traffic_source": "ncu dram__bytes_read+write per launch, mean over the launches of a token step "
                                           "(profiles/gemv_stream_*_decode_launches.md); null where no capture exists",
                         "peak_source": peak_src, "bytes_per_launch": alg / n_calls,
                         "us_per_launch": ms_step * 1e3 / n_calls, "launches_per_step": n_calls,
                         "note": "algorithmic bytes of one launch (mean over the step's launches) / mean launch duration "
                                 "from CUDA events around the graph-replayed step (inter-kernel gaps included)"},
            "correction_overhead": {"time_ratio": ms_step / ms_plain, "plain_ms_per_step": ms_plain,
                                    "byte_ratio_floor": alg / alg_plain},
            "prefill": prefill, "tp_parity": tp_par, "sweep": sweep}
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = gpu_arm_cpu_baseline(args, shape)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def measure_prefill(arm, stack, tokens, steps):
    torch = arm.torch
    with torch.cuda.stream(arm.stream):
        pplan = stack.plan(tokens, corrected=True, fuse_groups=not arm.args.unfused)
    ms_p, _ = arm.timed(stack, arm.make_step(stack, pplan), steps, 3, False)
    stack.check_status(pplan)
    fl = stack.algorithmic_flops(tokens, corrected=True)
    out = {"tokens": tokens, "ms": ms_p, "tokens_per_s": tokens / (ms_p * 1e-3), "tflops": fl / (ms_p * 1e-3) / 1e12,
           "kernel": "gemm_w4a16_kernel (tcgen05)", "flops_per_pass": fl}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            mp_ = json.load(f)
        out["frac_of_measured_bf16_burst"] = out["tflops"] / float(mp_["bf16_tflops"])
        out["frac_of_measured_bf16_sustained"] = out["tflops"] / float(mp_["bf16_tflops_sustained"])
    except Exception:  # noqa: BLE001
        pass
    out["frac_of_nominal_fp16_dense"] = out["tflops"] / 2250.0
    stack._plans.clear()
    return out


def host_entry_step(arm, stack, plan, steps):
    """tokens/s of the step when every group call is glowq_w4a16_group_forward_host: host x in, host outputs out."""
    import ctypes
    torch = arm.torch
    lib, check = stack.ext.lib, stack.ext.check
    calls = []
    for i in range(plan["n"]):
        c = plan["calls"][i]
        x_host = torch.randn(c.M, c.IC).to(torch.float16).pin_memory()
        outs = [torch.empty(c.M, c.members[j].OC, dtype=torch.float16).pin_memory() for j in range(c.n_members)]
        ptrs = (ctypes.c_void_p * c.n_members)(*[o.data_ptr() for o in outs])
        calls.append((c, x_host, outs, ptrs))
    bytes_in = sum(x.numel() * 2 for _, x, _, _ in calls)
    bytes_out = sum(o.numel() * 2 for _, _, outs, _ in calls for o in outs)

    def step():
        for c, x_host, _, ptrs in calls:
            check(lib.glowq_w4a16_group_forward_host(ctypes.byref(c), x_host.data_ptr(), ptrs), "group_forward_host")
    with torch.cuda.stream(arm.stream):
        step()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        ms = (time.perf_counter() - t0) / steps * 1e3
    return {"value": plan["M"] / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "h2d_bytes_per_step": bytes_in,
            "d2h_bytes_per_step": bytes_out, "calls_per_step": plan["n"],
            "path": "glowq_w4a16_group_forward_host per group (copy x in, launch, copy every output out, synchronise)"}


def build_dropin_model(stack):
    """The stack's linears behind the reference's own Python surface: a module tree with the artefact names
    (model.layers.{i}.self_attn.q_proj ...) whose leaves are CudaW4A16Linear shells over copies of the stack's packed
    tensors, patched by patch_svd_correction_wrappers from `shared` / `bmap` dicts in GlowQ's key scheme."""
    import torch.nn as nn
    import glowq_b200 as G
    root = nn.Module()
    root.model = nn.Module()
    layers = nn.ModuleList()
    shared, bmap = {}, {}
    n_layers = len(stack.groups) // 4
    for li in range(n_layers):
        qkv, o, mlp, down = stack.groups[4 * li:4 * li + 4]
        layer = nn.Module()
        layer.self_attn, layer.mlp = nn.Module(), nn.Module()
        for parent, grp, names, gk in ((layer.self_attn, qkv, ("q_proj", "k_proj", "v_proj"), f"layer{li}_qkv"),
                                       (layer.mlp, mlp, ("gate_proj", "up_proj"), f"layer{li}_mlp")):
            pname = "self_attn" if parent is layer.self_attn else "mlp"
            for name, m in zip(names, grp.members):
                setattr(parent, name, m.as_module())
                if grp.enabled:
                    shared[f"{gk}.B_shared"] = grp.R
                    shared[f"{gk}.{name}.A"] = m.L
                    bmap[f"model.layers.{li}.{pname}.{name}.weight"] = f"{gk}.B_shared"
        for parent, grp, name, pname in ((layer.self_attn, o, "o_proj", "self_attn"), (layer.mlp, down, "down_proj", "mlp")):
            setattr(parent, name, grp.members[0].as_module())
            if grp.enabled:
                mod = f"model.layers.{li}.{pname}.{name}"
                shared[f"{mod}.A"], shared[f"{mod}.B"] = grp.members[0].L, grp.R
                bmap[f"{mod}.weight"] = f"{mod}.B"
        layers.append(layer)
    root.model.layers = layers
    G.patch_svd_correction_wrappers_cumulative(root, shared, bmap, {k.rsplit(".", 1)[0] if k.endswith(".B") else
                                                                    k.replace(".B_shared", "") for k in bmap.values()}, 1.0)
    return root


def dropin_step(arm, stack, plan, steps):
    """tokens/s of the same token step issued through the drop-in modules (convert -> patch -> module calls in the
    order a decoder layer makes them: q, k, v, o, gate, up, down), eagerly from Python and replayed from a CUDA graph."""
    torch = arm.torch
    os.environ["W4A16_KERNEL_OUT_DTYPE"] = "fp16"       # what the reference's step3 sets before converting
    model = build_dropin_model(stack)
    x, xa, xi = plan["inputs"]["hidden"], plan["inputs"]["attn"], plan["inputs"]["inter"]
    calls = []
    for layer in model.model.layers:
        a, m = layer.self_attn, layer.mlp
        calls += [(a.q_proj, x), (a.k_proj, x), (a.v_proj, x), (a.o_proj, xa), (m.gate_proj, x), (m.up_proj, x),
                  (m.down_proj, xi)]

    def step():
        out = None
        for mod, inp in calls:
            out = mod(inp)
        return out

    def time_it(run, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(arm.stream)
        for _ in range(n):
            run()
        e1.record(arm.stream)
        arm.stream.synchronize()
        return e0.elapsed_time(e1) / n

    with torch.cuda.stream(arm.stream):
        for _ in range(3):
            step()
        arm.stream.synchronize()
        ms_eager = time_it(step, steps)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=arm.stream):
            step()
        for _ in range(3):
            graph.replay()
        arm.stream.synchronize()
        ms_graph = time_it(graph.replay, steps)
    M = plan["M"]
    launches = sum(1 for mod, _ in calls if getattr(mod, "group_launcher", None) is None
                   or mod.group_launcher.members[0] is mod)
    del model, calls, graph
    torch.cuda.empty_cache()
    return {"value": M / (ms_graph * 1e-3), "unit": UNIT, "ms_per_step": ms_graph,
            "eager_tokens_per_s": M / (ms_eager * 1e-3), "eager_ms_per_step": ms_eager, "launches_per_step": launches,
            "path": "convert_to_cuda_w4a16-style modules + patch_svd_correction_wrappers, 7 module calls per layer in "
                    "decoder order; `value` replays them from a CUDA graph, `eager_*` pays the Python dispatch"}


def run_sweep(arm, args, main_stack=None):
    """The other benchmark configurations, from the same process (one GPU): decode batches of the Llama-3.2-3B shape, the
    Qwen2.5-7B shape with a seeded 50 % GlowQ-S mask, the Llama-2-13B shape, and the isolated-linear token sweep on the
    Qwen3-14B shapes.  Short runs (20 timed steps each); every line carries its own roofline figures."""
    from glowq_b200.stack import SHAPES
    torch = arm.torch
    peak, _ = measured_peaks()
    out = {"decode": [], "qwen3_14b_m_sweep": []}
    steps = 20

    def decode_line(stack, shape, M, fraction):
        ms, _, plan = arm.decode(stack, M, steps, 3, corrected=True)
        alg = stack.algorithmic_bytes(M, corrected=True)
        fl = stack.algorithmic_flops(M, corrected=True)
        stack._plans.clear()
        return {"model": shape.name, "batch": M, "glowq_s_fraction": fraction, "ms_per_step": ms,
                "tokens_per_s": M / (ms * 1e-3), "GBs": alg / (ms * 1e-3) / 1e9, "frac_of_measured_hbm": alg / (ms * 1e-3) / 1e9 / peak,
                "tflops": fl / (ms * 1e-3) / 1e12, "kernel": "gemv_stream" if M <= 8 else "gemm_tcgen05",
                "launches": plan["n"]}

    for name, batches, fraction in (("llama-3.2-3b", (1, 8, 32), 1.0), ("qwen2.5-7b", (1, 64), 0.5),
                                    ("llama-2-13b", (1, 16, 64), 1.0)):
        shape = SHAPES[name]
        reuse = main_stack is not None and main_stack.shape.name == name and fraction >= 1.0
        stack = main_stack if reuse else arm.build_stack(shape, None, fraction)
        for M in batches:
            out["decode"].append(decode_line(stack, shape, M, fraction))
        del stack
        torch.cuda.empty_cache()
    # isolated corrected linears of one Qwen3-14B layer (two layer copies rotate so that every launch reads HBM up to
    # the token counts where the GEMM is compute-bound anyway)
    shape = SHAPES["qwen3-14b"]
    stack = arm.build_stack(shape, 2, 1.0)
    for M in (1, 2, 4, 8, 16, 32, 64, 128, 256, 1024, 4096):
        ms, _, plan = arm.decode(stack, M, 10 if M >= 1024 else steps, 3, corrected=True)
        alg = stack.algorithmic_bytes(M, corrected=True) / 2
        fl = stack.algorithmic_flops(M, corrected=True) / 2
        us = ms * 1e3 / 2
        out["qwen3_14b_m_sweep"].append({"M": M, "us_per_layer": us, "GBs": alg / us / 1e3, "tflops": fl / us / 1e6,
                                         "kernel": "gemv_stream" if M <= 8 else "gemm_tcgen05"})
        stack._plans.clear()
        torch.cuda.empty_cache()
    del stack
    torch.cuda.empty_cache()
    return out


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
