"""Packed checkpoints (glowq_b200.artifacts): a reloaded model must equal a freshly converted one bit for bit, with
or without correction wrappers, and the loader must refuse what does not fit.  CPU only: no kernel is launched."""
import copy

import pytest
import torch
import torch.nn as nn

from glowq_b200 import (AddSVDCorrection, CudaW4A16Linear, convert_to_cuda_w4a16, load_packed,
                        patch_svd_correction_wrappers, patch_svd_correction_wrappers_cumulative, save_packed)
from toy_model import ToyDecoder, make_artifacts

BUFS = ("qweight_i32", "qzeros_i32", "scales_f16")


def _packed_modules(model):
    out = {}
    for n, m in model.named_modules():
        if isinstance(m, CudaW4A16Linear):
            out[n[:-len(".inner")] if n.endswith(".inner") else n] = m
    return out


def _assert_same_packed(a, b):
    ma, mb = _packed_modules(a), _packed_modules(b)
    assert ma.keys() == mb.keys() and len(ma) > 0
    for n in ma:
        for buf in BUFS:
            ta, tb = getattr(ma[n], buf), getattr(mb[n], buf)
            assert ta.dtype == tb.dtype and ta.shape == tb.shape, (n, buf)
            assert torch.equal(ta, tb), (n, buf)
        assert (ma[n].bias is None) == (mb[n].bias is None)
        if ma[n].bias is not None:
            assert torch.equal(ma[n].bias, mb[n].bias)
        assert (ma[n].in_features, ma[n].out_features, ma[n].group_size) == \
               (mb[n].in_features, mb[n].out_features, mb[n].group_size)


@pytest.mark.parametrize("bias", [False, True])
def test_round_trip_equals_fresh_conversion(tmp_path, bias):
    src = ToyDecoder(n_layers=2, hidden=256, kv=128, inter=384, bias=bias, seed=3)
    converted = convert_to_cuda_w4a16(copy.deepcopy(src), 128)
    path = str(tmp_path / "packed.pt")
    assert save_packed(converted, path) == 14          # 2 layers x 7 projections; lm_head stays a float linear
    fresh = copy.deepcopy(src)
    loaded, shared, bmap = load_packed(fresh, path)
    assert shared is None and bmap is None
    _assert_same_packed(converted, loaded)
    assert isinstance(loaded.lm_head, nn.Linear)


def test_round_trip_with_input_width_that_is_not_a_whole_number_of_groups(tmp_path):
    """in_features = 200 with groups of 128: the quantiser pads to 256 columns (32 packed words), a fresh shell has
    ceil(200/8) = 25; the loader must take the stored, padded tensors as from_float does."""
    class Tiny(nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(5)
            self.proj = nn.Linear(200, 16, bias=True)

    src = Tiny()
    converted = convert_to_cuda_w4a16(copy.deepcopy(src), 128)
    assert tuple(converted.proj.qweight_i32.shape) == (16, 32)
    path = str(tmp_path / "ragged.pt")
    assert save_packed(converted, path) == 1
    loaded, _, _ = load_packed(copy.deepcopy(src), path)
    _assert_same_packed(converted, loaded)


def test_wrapped_model_saves_under_unwrapped_names_and_carries_the_low_rank_artifacts(tmp_path):
    src = ToyDecoder(n_layers=2, hidden=256, kv=128, inter=384, seed=4)
    shared, bmap = make_artifacts(src, rank=16)
    converted = convert_to_cuda_w4a16(copy.deepcopy(src), 128)
    patch_svd_correction_wrappers(converted, shared, bmap, alpha_svd=1.0)
    assert any(isinstance(m, AddSVDCorrection) for m in converted.modules())
    path = str(tmp_path / "packed_lr.pt")
    save_packed(converted, path, shared=shared, bmap=bmap)
    loaded, shared2, bmap2 = load_packed(copy.deepcopy(src), path)
    _assert_same_packed(converted, loaded)
    assert bmap2 == bmap and shared2.keys() == shared.keys()
    for k in shared:
        assert torch.equal(shared2[k], shared[k].cpu())
    # the reloaded model takes the patchers exactly like a converted one (GlowQ-S mask included)
    patch_svd_correction_wrappers_cumulative(loaded, shared2, bmap2, {"layer0_qkv", "layer1_mlp"}, alpha_svd=1.0)
    wrapped = sorted(n for n, m in loaded.named_modules() if isinstance(m, AddSVDCorrection))
    assert wrapped == sorted(f"model.layers.0.self_attn.{p}_proj" for p in "qkv") + \
                      sorted(f"model.layers.1.mlp.{p}_proj" for p in ("gate", "up"))


def test_loader_rejects_what_does_not_fit(tmp_path):
    src = ToyDecoder(n_layers=1, hidden=256, kv=128, inter=384, seed=5)
    path = str(tmp_path / "p.pt")
    save_packed(convert_to_cuda_w4a16(copy.deepcopy(src), 128), path)
    with pytest.raises(KeyError):                       # a linear of the model is not covered by the file
        load_packed(ToyDecoder(n_layers=2, hidden=256, kv=128, inter=384), path)
    with pytest.raises(ValueError):                     # same names, other sizes
        load_packed(ToyDecoder(n_layers=1, hidden=256, kv=128, inter=512), path)
    other = str(tmp_path / "other.pt")
    torch.save({"format": "something else"}, other)
    with pytest.raises(ValueError):
        load_packed(copy.deepcopy(src), other)
    with pytest.raises(ValueError):                     # nothing to save before conversion
        save_packed(copy.deepcopy(src), str(tmp_path / "none.pt"))
    # non-strict: a file covering fewer layers loads what it has
    loaded, _, _ = load_packed(ToyDecoder(n_layers=2, hidden=256, kv=128, inter=384), path, strict=False)
    assert isinstance(loaded.model.layers[0].mlp.down_proj, CudaW4A16Linear)
    assert isinstance(loaded.model.layers[1].mlp.down_proj, nn.Linear)
