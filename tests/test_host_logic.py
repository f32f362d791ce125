"""Host side of the drop-in (quantiser, conversion pass, wrappers, patchers, C-ABI exports) on CPU."""
import json
import os
import re

import numpy as np
import pytest
import torch

import glowq_oracle as O
from toy_model import ToyDecoder, make_artifacts

import glowq_b200
from glowq_b200 import (AddSVDCorrection, CudaW4A16Linear, MiniGroupCache, convert_to_cuda_w4a16,
                        patch_svd_correction_wrappers, patch_svd_correction_wrappers_cumulative)
from glowq_b200.cuda_w4a16 import kernels as K
from glowq_b200.cuda_w4a16.linear import _pack_int4_to_int32, _quantize_per_group_w4, _unpack_int4_i32

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
QUANT_TAGS = ["a", "ragged", "g10", "g32", "g9", "edge"]


@pytest.mark.parametrize("tag", QUANT_TAGS)
def test_quantiser_matches_reference_vectors(golden_quant, tag):
    g = golden_quant
    oc, ic, gs, icp = (int(v) for v in g[f"{tag}.meta"])
    qw, qz, sc, icp2 = _quantize_per_group_w4(torch.from_numpy(g[f"{tag}.w"]), gs)
    assert icp2 == icp
    np.testing.assert_array_equal(qw.numpy(), g[f"{tag}.qweight"])
    np.testing.assert_array_equal(qz.numpy(), g[f"{tag}.qzeros"])
    np.testing.assert_array_equal(sc.numpy().view(np.uint16), g[f"{tag}.scales"].view(np.uint16))


def test_quantiser_matches_oracle_random():
    rng = np.random.default_rng(5)
    for oc, ic, gs in [(3, 128, 128), (5, 200, 64), (16, 384, 128), (2, 8, 8), (7, 1032, 128)]:
        w = (rng.standard_normal((oc, ic)) * 0.02).astype(np.float16)
        a = _quantize_per_group_w4(torch.from_numpy(w), gs)
        b = O.quantize_per_group_w4(w, gs)
        for x, y in zip(a[:3], b[:3]):
            np.testing.assert_array_equal(x.numpy().view(np.uint8), np.ascontiguousarray(y).view(np.uint8))
        assert a[3] == b[3]


def test_pack_unpack():
    u4 = torch.randint(0, 16, (4, 6, 8), dtype=torch.uint8)
    packed = _pack_int4_to_int32(u4)
    np.testing.assert_array_equal(packed.numpy(), O.pack_int4_to_int32(u4.numpy()))
    np.testing.assert_array_equal(_unpack_int4_i32(packed, 48).numpy(), u4.reshape(4, 48).numpy())
    with pytest.raises(ValueError):
        _quantize_per_group_w4(torch.zeros(2, 12, dtype=torch.float16), 12)


def test_module_surface_and_state_dict():
    with pytest.raises(ValueError):
        CudaW4A16Linear(64, 8, group_size=12)
    lin = torch.nn.Linear(200, 24, bias=True).half()
    mod = CudaW4A16Linear.from_float(lin, 128)
    assert (mod.in_features, mod.out_features, mod.group_size, mod.groups, mod.groups_packed) == (200, 24, 128, 2, 1)
    assert mod.qweight_i32.shape == (24, 32) and mod.qzeros_i32.shape == (24, 1) and mod.scales_f16.shape == (24, 2)
    assert set(mod.state_dict()) == {"qweight_i32", "qzeros_i32", "scales_f16", "bias"}
    assert mod.gid.shape == (200,) and "gid" not in mod.state_dict()
    assert "in_features=200" in repr(mod)
    with pytest.raises(RuntimeError, match="CUDA"):
        mod(torch.zeros(1, 200, dtype=torch.float16))          # no CPU path
    with pytest.raises(ValueError, match="Input dim mismatch"):
        mod(torch.zeros(1, 100, dtype=torch.float16))


def _describe(model):
    rows, caches = {}, {}
    for name, mod in model.named_modules():
        if isinstance(mod, AddSVDCorrection):
            cid = None
            if mod.group_cache is not None:
                cid = caches.setdefault(id(mod.group_cache), len(caches))
            rows[name] = {"role": mod.role, "is_group": bool(mod.is_group), "cache": cid, "alpha": float(mod.alpha_svd),
                          "A": list(mod.A_q.shape), "B": list(mod.B_q.shape), "inner": type(mod.inner).__name__}
    kinds = {n: type(m).__name__ for n, m in model.named_modules() if isinstance(m, (torch.nn.Linear, CudaW4A16Linear))}
    return {"wrapped": rows, "linear_kinds": kinds}


def test_conversion_pass_matches_reference(golden_patch):
    model = convert_to_cuda_w4a16(ToyDecoder(), 128)
    assert _describe(model) == golden_patch["convert"]
    assert isinstance(model.lm_head, torch.nn.Linear)
    assert model._w4a16_conversion_errors == {}


def test_patch_all_matches_reference(golden_patch):
    model = convert_to_cuda_w4a16(ToyDecoder(), 128)
    shared, bmap = make_artifacts(model)
    patch_svd_correction_wrappers(model, shared, bmap, 1.0)
    assert _describe(model) == golden_patch["patch_all"]


def test_patch_damaged_artifacts_matches_reference(golden_patch):
    model = convert_to_cuda_w4a16(ToyDecoder(), 128)
    shared, bmap = make_artifacts(model)
    del shared["layer0_qkv.k_proj.A"]
    del shared["model.layers.1.mlp.down_proj.B"]
    bmap["model.layers.7.mlp.down_proj.weight"] = "model.layers.1.self_attn.o_proj.B"
    patch_svd_correction_wrappers(model, shared, bmap, 0.25)
    assert _describe(model) == golden_patch["patch_damaged"]


@pytest.mark.parametrize("tag", ["none", "qkv0_mlp1", "solo", "all"])
def test_glowq_s_mask_matches_reference(golden_patch, tag):
    case = golden_patch[f"mask.{tag}"]
    model = convert_to_cuda_w4a16(ToyDecoder(), 128)
    shared, bmap = make_artifacts(model)
    patch_svd_correction_wrappers_cumulative(model, shared, bmap, set(case["groups"]), 1.0)
    got = _describe(model)
    assert got["wrapped"] == case["wrapped"] and got["linear_kinds"] == case["linear_kinds"]


def test_wrapper_protocol_against_reference_trace(golden_forward, monkeypatch):
    """Role / cache behaviour with the launch stubbed out: which launches compute r and which load it must
    follow the cache states recorded from the reference wrapper."""
    calls = []

    def fake_launch(self, x2d, *, L=None, R=None, r_buf=None, r_mode=K.R_NONE, alpha=0.0):
        calls.append((r_mode, alpha, None if r_buf is None else r_buf.data_ptr()))
        return torch.zeros(x2d.size(0), self.out_features)

    monkeypatch.setattr(CudaW4A16Linear, "launch", fake_launch)
    monkeypatch.setattr(CudaW4A16Linear, "_flatten_input", lambda self, x: x.reshape(-1, x.shape[-1]))
    trace = json.loads(str(golden_forward["qkv2048.trace.M1.fp16.a1.0"]))
    cache = MiniGroupCache()
    x = torch.zeros(1, 64, dtype=torch.float16)
    mods = {}
    for name, role, *_ in trace:
        mods[name] = AddSVDCorrection(CudaW4A16Linear(64, 16), torch.zeros(16, 8), torch.zeros(8, 64), role, True, cache, 1.0)
    model = O.GroupCacheModel()
    for name, role, v0, u0, v1, u1 in trace:
        assert (int(cache.valid), cache.uses_left) == (v0, u0)
        mods[name](x)
        want = model.step(role)
        assert (int(cache.valid), cache.uses_left) == (v1, u1)
        assert calls[-1][0] == (K.R_COMPUTE if want == "compute" else K.R_LOAD)
    assert calls[0][2] == calls[1][2] == calls[2][2]          # k and v read the buffer q wrote
    # consumer without producer recomputes into a private buffer; alpha 0 short-circuits to the bare linear
    calls.clear()
    mods["k_proj"](x)
    assert calls[-1][0] == K.R_COMPUTE
    mods["k_proj"].alpha_svd = 0.0
    mods["k_proj"](x)
    assert calls[-1][0] == K.R_NONE
    # a different input tensor is a miss even when the cache is armed
    mods["q_proj"](x)
    mods["k_proj"].alpha_svd = 1.0
    mods["k_proj"](torch.ones(1, 64, dtype=torch.float16))
    assert calls[-1][0] == K.R_COMPUTE


def test_wrapper_rejects_foreign_inner_and_flags_mismatch():
    with pytest.raises(TypeError):
        AddSVDCorrection(torch.nn.Linear(4, 4), torch.zeros(4, 2), torch.zeros(2, 4), "solo", False, None)
    with pytest.warns(UserWarning):
        w = AddSVDCorrection(CudaW4A16Linear(64, 16), torch.zeros(8, 4), torch.zeros(4, 64), "solo", False, None)
    assert w._mismatch


def test_abi_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "glowq_w4a16.h")).read()
    declared = sorted(set(re.findall(r"\b(glowq_w4a16_[a-z_0-9]+)\s*\(", header)))
    assert declared, "no declarations found"
    ext = glowq_b200.load_w4a16_extension()
    for name in declared:
        assert hasattr(ext.lib, name), name
    assert set(declared) == set(K.EXPORTS)
    assert ext.lib.glowq_w4a16_version() == K.ABI_VERSION
    assert b"sm_100" in ext.lib.glowq_w4a16_strerror(5)
    # struct layouts agree with the header (sizes from the C side are fixed by the field lists)
    assert K.Member._fields_[0][0] == "qweight" and K.Group._fields_[-1][0] == "members"
    assert ext.workspace_bytes(1, 2048, 2048, 64, 1) >= 256


def test_workspace_sizes_cover_what_the_kernels_plan():
    """glowq_w4a16_workspace_bytes is host arithmetic (no GPU): it must grow with what a call may need - R-unit slots
    with the rank, K-slice slots for 9..256 tokens when the tiles cannot fill the SMs, the sliced last wave above
    256 tokens - and stay small for decode-sized calls."""
    from glowq_b200.cuda_w4a16 import kernels as K
    ext = K.load_w4a16_extension()
    wb = ext.workspace_bytes
    assert wb(0, 3072, 3072, 0, 1) == 256 and wb(1, 0, 3072, 0, 1) == 256          # nothing to do: header only
    assert all(wb(m, 3072, 3072, 64, 1) % 256 == 0 for m in (1, 8, 33, 300))
    # decode: counters + R-unit slots, well under a megabyte for the Llama-3.2-3B shapes
    assert wb(1, 3072, 5120, 0, 3) < wb(1, 3072, 5120, 64, 3) < (1 << 20)
    assert wb(1, 3072, 5120, 64, 3) <= wb(1, 3072, 5120, 256, 3)
    # 17..256 tokens: fp32 partial tiles of the K-sliced GEMM for a launch with few tiles ...
    small, mid = wb(8, 8192, 3072, 0, 1), wb(32, 8192, 3072, 0, 1)
    assert mid > small and mid >= 12 * 8 * 2 * 32 * 128 * 4        # 12 tiles x 8 slices x 2 x 32 rows x 128 columns
    # ... from 9 tokens on, where the automatic choice takes the GEMM (a launch of 9..16 tokens without slot space
    # would walk all of K in one CTA per tile)
    assert wb(9, 8192, 3072, 0, 1) == wb(16, 8192, 3072, 0, 1) == mid
    # ... but not for one whose tiles already fill the SMs (2 x 17408 output columns = 136 tiles of 256)
    assert wb(32, 5120, 34816, 0, 2) < (1 << 20)
    # above 256 tokens: room for the sliced last wave (64 slots of a 256 x 256 fp32 tile)
    assert wb(2048, 3072, 5120, 0, 3) >= 64 * 256 * 256 * 4
    assert wb(2048, 3072, 5120, 64, 3) >= wb(2048, 3072, 5120, 0, 3)


def test_workspace_covers_every_k_sliced_plan():
    """For 9..256 tokens the GEMM may cut K into slices whose fp32 partial tiles live at the end of the workspace; the
    size the library reports must cover the plan for either column-tile width (restated here from the host code)."""
    from glowq_b200.cuda_w4a16 import kernels as K
    wb = K.load_w4a16_extension().workspace_bytes
    cdiv = lambda a, b: -(-a // b)
    sms = 148
    for ocs in ([3072], [3072, 1024, 1024], [8192, 8192], [5120], [5120, 1024, 1024], [17408, 17408], [384], [136, 200]):
        for ic in (1024, 3072, 8192, 17408):
            for m in (9, 16, 17, 32, 64, 100, 128, 129, 200, 256):
                need = 0
                for nn in (1, 2):
                    tiles = sum(cdiv(oc, 128 * nn) for oc in ocs) * cdiv(m, 128)
                    ks = max(1, min(8, sms // tiles, cdiv(ic, 64) // 8)) if tiles * 2 <= sms else 1
                    if ks > 1:
                        rows = min(128, cdiv(m, 32) * 32)
                        need = max(need, ks * tiles * nn * rows * 128 * 4)
                have = wb(m, ic, sum(ocs), 0, len(ocs))
                assert have >= need + 256, (ocs, ic, m, have, need)
