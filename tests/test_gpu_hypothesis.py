"""Randomised shapes (hypothesis) through the C ABI: bit-exact dequantisation and forward parity for layouts the
hand-picked cases do not cover - odd output counts, ragged input widths, group counts that are not multiples of 8,
small group sizes (generic kernel), 1..24 tokens, optional bias and correction."""
import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings, strategies as st

import glowq_oracle as O
from glowq_b200.cuda_w4a16 import kernels as K
from gpu_helpers import Linear, assert_close, dev, ext, make_group, new_out, run_group, status_ok

pytestmark = pytest.mark.gpu
COMMON = dict(max_examples=25, deadline=None, suppress_health_check=[HealthCheck.too_slow, HealthCheck.data_too_large])


@settings(**COMMON)
@given(oc=st.integers(1, 200), words=st.integers(1, 90), gs=st.sampled_from([8, 16, 32, 64, 128]), seed=st.integers(0, 2**16))
def test_dequant_bit_exact_random_layouts(oc, words, gs, seed):
    ic = words * 8
    rng = np.random.default_rng(seed)
    lin = Linear(rng, oc, ic, gs, w_std=0.03)
    got = ext().dequant(lin.d_qweight, lin.d_scales, lin.d_qzeros, ic, gs)
    want = O.dequant_full(lin.qweight, lin.qzeros, lin.scales, ic, gs)
    np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), want.view(np.uint16))


@settings(**COMMON)
@given(oc=st.integers(1, 300), ic8=st.integers(16, 400), M=st.integers(1, 24), rank8=st.integers(0, 12),
       bias=st.booleans(), gs=st.sampled_from([128, 128, 128, 64]), seed=st.integers(0, 2**16))
def test_forward_parity_random_layouts(oc, ic8, M, rank8, bias, gs, seed):
    ic, rank = ic8 * 8, rank8 * 8
    rng = np.random.default_rng(seed)
    lin = Linear(rng, oc, ic, gs, bias=bias, rank=rank)
    x = rng.standard_normal((M, ic)).astype(np.float16)
    out = new_out(M, lin)
    if rank:
        R = (rng.standard_normal((rank, ic)) * 0.01).astype(np.float16)
        r_buf = torch.zeros(M, rank, dtype=torch.float16, device="cuda")
        g = make_group(dev(x), [lin], [out], R_d=dev(R), r_buf=r_buf, r_mode=K.R_COMPUTE, alpha=0.75)
        want = lin.oracle(x, R, alpha=0.75)
    else:
        g = make_group(dev(x), [lin], [out])
        want = lin.oracle(x)
    assert run_group(g) == 0 and status_ok(g) == 0
    # tiny outputs (few input columns) make the relative figure meaningless: bound it by the absolute tolerance too
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    ma, mr = O.parity_errors(got, want)
    assert ma <= 2e-2 and (mr <= 1e-3 or ma <= 2e-3), (ma, mr)
