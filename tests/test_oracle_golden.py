"""The CPU oracle against outputs of GlowQ's own code (tests/golden/, made by make_golden.py)."""
import json

import numpy as np
import pytest

import glowq_oracle as O

QUANT_TAGS = ["a", "ragged", "g10", "g32", "g9", "edge"]


@pytest.mark.parametrize("tag", QUANT_TAGS)
def test_quantiser_bit_exact(golden_quant, tag):
    g = golden_quant
    oc, ic, gs, icp = (int(v) for v in g[f"{tag}.meta"])
    qw, qz, sc, icp2 = O.quantize_per_group_w4(g[f"{tag}.w"], gs)
    assert icp2 == icp
    np.testing.assert_array_equal(qw, g[f"{tag}.qweight"])
    np.testing.assert_array_equal(qz, g[f"{tag}.qzeros"])
    np.testing.assert_array_equal(sc.view(np.uint16), g[f"{tag}.scales"].view(np.uint16))


@pytest.mark.parametrize("tag", QUANT_TAGS)
def test_dequant_bit_exact(golden_quant, tag):
    g = golden_quant
    oc, ic, gs, icp = (int(v) for v in g[f"{tag}.meta"])
    deq = O.dequant_full(g[f"{tag}.qweight"], g[f"{tag}.qzeros"], g[f"{tag}.scales"], ic, gs)
    np.testing.assert_array_equal(deq.view(np.uint16), g[f"{tag}.deq"].view(np.uint16))


def test_pack_unpack_roundtrip():
    rng = np.random.default_rng(0)
    u4 = rng.integers(0, 16, size=(5, 7, 8), dtype=np.uint8)
    packed = O.pack_int4_to_int32(u4)
    assert packed.dtype == np.int32 and (packed < 0).any()
    back = O.unpack_int4_i32(packed.reshape(5, 7), 56)
    np.testing.assert_array_equal(back, u4.reshape(5, 56))


@pytest.mark.parametrize("tag,d,rank,bias", [("qkv2048", 2048, 64, False), ("qkv1152b", 1152, 32, True)])
@pytest.mark.parametrize("M", [1, 16])
@pytest.mark.parametrize("alpha", [1.0, 0.5, 0.0])
def test_forward_oracle_vs_reference_module(golden_forward, tag, d, rank, bias, M, alpha):
    """fp32 oracle vs the reference's module path (fp32 and fp16 output dtypes): inside the
    stated tolerances, and tighter for the fp32-output run."""
    g = golden_forward
    x = g[f"{tag}.x{M}"]
    R = g[f"{tag}.R"]
    for n in ("q_proj", "k_proj", "v_proj"):
        deq = O.dequant_full(g[f"{tag}.{n}.qweight"], g[f"{tag}.{n}.qzeros"], g[f"{tag}.{n}.scales"], d, 128)
        b = g[f"{tag}.{n}.bias"] if bias else None
        y = O.corrected_forward_fp32(x, deq, R, g[f"{tag}.{n}.L"], alpha, b)
        for od, tol_abs, tol_rel in (("fp32", 4e-3, 1e-3), ("fp16", 2e-2, 1e-3)):
            yref = g[f"{tag}.y.M{M}.{od}.a{alpha}.{n}"]
            assert yref.shape == y.shape
            ma, mr = O.parity_errors(yref, y)
            assert ma <= tol_abs and mr <= tol_rel, (n, od, ma, mr)
            yr = O.reference_rounded_forward(x, deq, R, g[f"{tag}.{n}.L"], alpha, b,
                                             np.float16 if od == "fp16" else np.float32)
            ma2, _ = O.parity_errors(yref, yr)
            assert ma2 <= 4e-3, (n, od, ma2)


@pytest.mark.parametrize("alpha", [1.0, 0.5])
def test_cache_protocol_trace(golden_forward, alpha):
    trace = json.loads(str(golden_forward[f"qkv2048.trace.M1.fp16.a{alpha}"]))
    model = O.GroupCacheModel()
    for name, role, v0, u0, v1, u1 in trace:
        assert O.role_from_suffix(name) == role
        assert (int(model.valid), model.uses_left) == (v0, u0)
        model.step(role)
        assert (int(model.valid), model.uses_left) == (v1, u1)


def test_cache_model_miss_and_gate():
    m = O.GroupCacheModel()
    assert m.step("k") == "compute"            # consumer before producer recomputes
    assert m.step("gate") == "compute" and m.uses_left == 1
    assert m.step("up") == "hit" and not m.valid
    assert m.step("up") == "compute"
    assert m.step("solo", is_group=False) == "compute"


def test_c_oracle_matches_numpy(golden_forward, golden_quant):
    import c_oracle as C
    g = golden_quant
    for tag in QUANT_TAGS:
        oc, ic, gs, icp = (int(v) for v in g[f"{tag}.meta"])
        deq = C.dequant(g[f"{tag}.qweight"], g[f"{tag}.scales"], g[f"{tag}.qzeros"], ic, gs)
        np.testing.assert_array_equal(deq.view(np.uint16), g[f"{tag}.deq"].view(np.uint16))
    f = golden_forward
    tag, d = "qkv1152b", 1152
    x, R = f[f"{tag}.x16"], f[f"{tag}.R"]
    r_io = np.zeros((16, R.shape[0]), np.float32)
    for i, n in enumerate(("q_proj", "k_proj", "v_proj")):
        args = (f[f"{tag}.{n}.qweight"], f[f"{tag}.{n}.scales"], f[f"{tag}.{n}.qzeros"])
        deq = O.dequant_full(args[0], args[2], args[1], d, 128)
        want = O.corrected_forward_fp32(x, deq, R, f[f"{tag}.{n}.L"], 0.5, f[f"{tag}.{n}.bias"])
        got = C.corrected_forward(x, *args, 128, bias=f[f"{tag}.{n}.bias"], R=R, L=f[f"{tag}.{n}.L"],
                                  alpha=0.5, r_io=r_io, r_mode=1 if i == 0 else 2)
        ma, mr = O.parity_errors(got, want)
        assert ma < 1e-4 and mr < 1e-5, (n, ma, mr)


def test_residual_rmsnorm_matches_the_model_code():
    """The oracle's residual add + RMSNorm against the module the reference's model code runs (HF LlamaRMSNorm on
    CPU, fp16 in / fp16 out), bit for bit up to the last-place differences of the fp32 mean."""
    import torch
    from transformers.models.llama.modeling_llama import LlamaRMSNorm
    rng = np.random.default_rng(21)
    for M, d in ((1, 256), (5, 3072)):
        x = rng.standard_normal((M, d)).astype(np.float16)
        res = (rng.standard_normal((M, d)) * 3).astype(np.float16)
        w = (1 + 0.1 * rng.standard_normal(d)).astype(np.float16)
        norm = LlamaRMSNorm(d, eps=1e-5)
        norm.weight.data = torch.from_numpy(w.copy())
        h_t = torch.from_numpy(res.copy()) + torch.from_numpy(x.copy())
        want = norm(h_t).detach().numpy()
        got, h = O.residual_rmsnorm_f16(x, res, w, 1e-5)
        assert np.array_equal(h.view(np.uint16), h_t.numpy().view(np.uint16))
        diff = np.abs(got.astype(np.float32) - want.astype(np.float32))
        assert (diff <= np.abs(want.astype(np.float32)) * 2 ** -9 + 1e-7).all()       # at most one fp16 ulp
        assert (got.view(np.uint16) != want.view(np.uint16)).mean() < 0.02
