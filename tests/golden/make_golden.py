"""Generate the golden fixtures in this directory by running GlowQ's own Python code.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/GLOWQ        (or GLOWQ_REFERENCE=/path/to/GLOWQ)

It imports the reference in place (nothing is copied), runs its quantiser, its pure-torch
dequantiser, its replacement module and its correction wrapper / patchers on seeded CPU
inputs, and stores inputs and outputs as ``.npz`` / ``.json`` files.  The tests only read
those files; they never need the reference checkout.
"""
import json
import os
import sys
import types

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("GLOWQ_REFERENCE", "")
if not os.path.isdir(os.path.join(REF, "src", "cuda_w4a16")):
    sys.exit("usage: make_golden.py /path/to/GLOWQ  (a checkout of the reference with src/cuda_w4a16)")
HERE = os.path.dirname(os.path.abspath(__file__))
os.environ.update(DISABLE_TRITON="1", W4A16_FORCE_GEMM="1", W4A16_GEMM_CUDA="0")
sys.path.insert(0, os.path.join(REF, "src"))
sys.path.insert(0, os.path.join(REF, "src", "restoration"))
sys.path.insert(0, os.path.dirname(HERE))

import numpy as np
import torch

torch.set_num_threads(4)
from cuda_w4a16.linear import CudaW4A16Linear, _quantize_per_group_w4, convert_to_cuda_w4a16  # noqa: E402
import step3_eval_dataset as s3  # noqa: E402

from toy_model import ToyDecoder, make_artifacts  # noqa: E402


def npy(t):
    return t.detach().cpu().numpy()


# ---------------------------------------------------------------- 1. quantiser + dequantiser
def quant_cases():
    out = {}
    g = torch.Generator().manual_seed(0)
    shapes = [("a", 24, 256, 128), ("ragged", 8, 136, 128), ("g10", 16, 1280, 128),
              ("g32", 8, 64, 32), ("g9", 8, 1152, 128), ("edge", 6, 256, 128)]
    for tag, oc, ic, gs in shapes:
        w = (torch.randn(oc, ic, generator=g) * 0.02).to(torch.float16)
        if tag == "edge":   # constant, all-zero, one-sided and large-magnitude groups
            w[0, :128] = 0.5
            w[1, :128] = 0.0
            w[2, :128] = -0.25
            w[3] = w[3].abs()
            w[4] = -w[4].abs()
            w[5] = w[5] * 1000
        lin = torch.nn.Linear(ic, oc, bias=False).half()
        lin.weight.data.copy_(w)
        mod = CudaW4A16Linear.from_float(lin, gs)
        qw, qz, sc, icp = _quantize_per_group_w4(w, gs)
        assert torch.equal(qw, mod.qweight_i32) and torch.equal(qz, mod.qzeros_i32)
        deq = mod._dequant_full_weight_fallback()
        out[f"{tag}.w"] = npy(w)
        out[f"{tag}.meta"] = np.array([oc, ic, gs, icp], dtype=np.int64)
        out[f"{tag}.qweight"] = npy(qw)
        out[f"{tag}.qzeros"] = npy(qz)
        out[f"{tag}.scales"] = npy(sc)
        out[f"{tag}.deq"] = npy(deq)
    np.savez_compressed(os.path.join(HERE, "quant_cases.npz"), **out)
    print("quant_cases.npz", len(out))


# ---------------------------------------------------------------- 2. corrected forward
def forward_cases():
    """OPT-1.3B-shaped QKV group cut down to 64 output rows per member (d = 2048, g = 128,
    rank 64, M in {1, 16}) plus a biased, ragged-G group (d = 1152 -> G = 9)."""
    out = {}
    for tag, d, ocs, rank, bias in (("qkv2048", 2048, (64, 64, 64), 64, False),
                                   ("qkv1152b", 1152, (48, 16, 16), 32, True)):
        gw = torch.Generator().manual_seed(0)
        gf = torch.Generator().manual_seed(1)
        gx = torch.Generator().manual_seed(2)
        names = ("q_proj", "k_proj", "v_proj")
        mods = []
        for oc in ocs:
            lin = torch.nn.Linear(d, oc, bias=bias).half()
            lin.weight.data.copy_((torch.randn(oc, d, generator=gw) * 0.02).half())
            if bias:
                lin.bias.data.copy_((torch.randn(oc, generator=gw) * 0.1).half())
            mods.append(CudaW4A16Linear.from_float(lin, 128))
        R = (torch.randn(rank, d, generator=gf) * 0.01).half()
        Ls = [(torch.randn(oc, rank, generator=gf) * 0.01).half() for oc in ocs]
        out[f"{tag}.R"] = npy(R)
        for n, m, L in zip(names, mods, Ls):
            out[f"{tag}.{n}.qweight"] = npy(m.qweight_i32)
            out[f"{tag}.{n}.qzeros"] = npy(m.qzeros_i32)
            out[f"{tag}.{n}.scales"] = npy(m.scales_f16)
            out[f"{tag}.{n}.L"] = npy(L)
            if bias:
                out[f"{tag}.{n}.bias"] = npy(m.bias.data)
        for M in (1, 16):
            x = torch.randn(M, d, generator=gx).half()
            out[f"{tag}.x{M}"] = npy(x)
            for od in ("fp16", "fp32"):
                os.environ["W4A16_KERNEL_OUT_DTYPE"] = od
                for alpha in (1.0, 0.5, 0.0):
                    cache = s3.MiniGroupCache()
                    trace = []
                    for n, m, L in zip(names, mods, Ls):
                        role = s3._role_from_suffix(n)
                        w = s3.AddSVDCorrection(m, L, R, role, True, cache, alpha)
                        before = (cache.valid, cache.uses_left)
                        y = w(x)
                        trace.append([n, role, int(before[0]), before[1], int(cache.valid), cache.uses_left])
                        out[f"{tag}.y.M{M}.{od}.a{alpha}.{n}"] = npy(y)
                    out[f"{tag}.trace.M{M}.{od}.a{alpha}"] = np.array(json.dumps(trace))
    np.savez_compressed(os.path.join(HERE, "forward_cases.npz"), **out)
    print("forward_cases.npz", len(out))


# ---------------------------------------------------------------- 3. conversion pass + patchers
WRAPPER_TYPES = [s3.AddSVDCorrection]   # the GlowQ-S script brings its own copy of the class


def describe(model):
    rows = {}
    caches = {}
    for name, mod in model.named_modules():
        if isinstance(mod, tuple(WRAPPER_TYPES)):
            cid = None
            if mod.group_cache is not None:
                cid = caches.setdefault(id(mod.group_cache), len(caches))
            rows[name] = {"role": mod.role, "is_group": bool(mod.is_group), "cache": cid,
                          "alpha": float(mod.alpha_svd), "A": list(mod.A_q.shape), "B": list(mod.B_q.shape),
                          "inner": type(mod.inner).__name__}
    kinds = {n: type(m).__name__ for n, m in model.named_modules()
             if isinstance(m, (torch.nn.Linear, CudaW4A16Linear))}
    return {"wrapped": rows, "linear_kinds": kinds}


def patch_cases():
    # the GlowQ-S patcher module plots with matplotlib/seaborn, which are only needed for figures
    for name in ("matplotlib", "matplotlib.pyplot", "seaborn"):
        sys.modules.setdefault(name, types.ModuleType(name))
    os.environ.pop("DISABLE_TRITON", None)   # its TritonTrue4BitLinear class needs the triton import
    import step4_evaluate_cumulative as s4
    os.environ["DISABLE_TRITON"] = "1"
    WRAPPER_TYPES.append(s4.AddSVDCorrection)

    result = {}
    model = convert_to_cuda_w4a16(ToyDecoder(), 128)
    shared, bmap = make_artifacts(model)
    result["convert"] = describe(model)
    s3.patch_svd_correction_wrappers(model, shared, bmap, 1.0)
    result["patch_all"] = describe(model)

    # damaged artefacts: a missing A, a missing B and a name that is not in the model
    model = convert_to_cuda_w4a16(ToyDecoder(), 128)
    shared2 = dict(shared)
    del shared2["layer0_qkv.k_proj.A"]
    del shared2["model.layers.1.mlp.down_proj.B"]
    bmap2 = dict(bmap)
    bmap2["model.layers.7.mlp.down_proj.weight"] = "model.layers.1.self_attn.o_proj.B"
    s3.patch_svd_correction_wrappers(model, shared2, bmap2, 0.25)
    result["patch_damaged"] = describe(model)

    masks = {"none": [], "qkv0_mlp1": ["layer0_qkv", "layer1_mlp"],
             "solo": ["model.layers.0.self_attn.o_proj", "model.layers.1.mlp.down_proj"],
             "all": sorted({(b.replace(".B_shared", "") if "B_shared" in b else b.rsplit(".", 1)[0])
                            for b in bmap.values()})}
    for tag, groups in masks.items():
        model = convert_to_cuda_w4a16(ToyDecoder(), 128)
        s4.patch_svd_correction_wrappers_cumulative(model, shared, bmap, set(groups), 1.0)
        result[f"mask.{tag}"] = {"groups": groups, **describe(model)}
    with open(os.path.join(HERE, "patch_cases.json"), "w") as f:
        json.dump(result, f, indent=1, sort_keys=True)
    print("patch_cases.json", list(result))

    # full toy forward through the patched model's wrappers, HF call order, fp16 output
    os.environ["W4A16_KERNEL_OUT_DTYPE"] = "fp16"
    model = convert_to_cuda_w4a16(ToyDecoder(), 128)
    s3.patch_svd_correction_wrappers(model, shared, bmap, 1.0)
    gx = torch.Generator().manual_seed(2)
    out = {}
    for M in (1, 5):
        x = torch.randn(M, 256, generator=gx).half()
        xi = torch.randn(M, 384, generator=gx).half()
        out[f"x{M}"] = npy(x)
        out[f"xi{M}"] = npy(xi)
        for li in range(2):
            for p in ToyDecoder.PROJ:
                inp = xi if p.endswith("down_proj") else x
                out[f"y{M}.{li}.{p}"] = npy(model.proj(li, p)(inp))
    np.savez_compressed(os.path.join(HERE, "toy_forward.npz"), **out)
    print("toy_forward.npz", len(out))


if __name__ == "__main__":
    quant_cases()
    forward_cases()
    patch_cases()
