"""CUDA path vs the CPU oracle through the C ABI (needs a B200).  Tolerances: dequantised weights bit-exact;
outputs within max-abs 2e-2 and mean-rel 1e-3 of the fp32 oracle."""
import ctypes
import json

import numpy as np
import pytest
import torch

import c_oracle as C
import glowq_oracle as O
from glowq_b200.cuda_w4a16 import kernels as K
from gpu_helpers import (Linear, assert_close, dev, ext, make_group, new_out, run_group, status_ok, TOL_ABS, TOL_REL)

pytestmark = pytest.mark.gpu
QUANT_TAGS = ["a", "ragged", "g10", "g32", "g9", "edge"]


# ---------------------------------------------------------------------------------------------- dequant
@pytest.mark.parametrize("tag", QUANT_TAGS)
def test_dequant_bit_exact_golden(golden_quant, tag):
    g = golden_quant
    oc, ic, gs, icp = (int(v) for v in g[f"{tag}.meta"])
    got = ext().dequant(dev(g[f"{tag}.qweight"]), dev(g[f"{tag}.scales"]), dev(g[f"{tag}.qzeros"]), ic, gs)
    np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), g[f"{tag}.deq"].view(np.uint16))


@pytest.mark.parametrize("oc,ic,gs", [(512, 4096, 128), (100, 520, 8), (3072, 8192, 128), (33, 264, 24)])
def test_dequant_bit_exact_random(oc, ic, gs):
    rng = np.random.default_rng(oc + ic)
    lin = Linear(rng, oc, ic, gs, w_std=0.05)
    got = ext().dequant(lin.d_qweight, lin.d_scales, lin.d_qzeros, ic, gs)
    want = O.dequant_full(lin.qweight, lin.qzeros, lin.scales, ic, gs)
    np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), want.view(np.uint16))


def test_dequant_all_codes_and_zeros_exhaustive():
    """Every (code, zero) pair with awkward scales, including subnormal products."""
    scales = np.array([1.0, 0.00731, 6.1e-5, 6e-8, 123.5, 0.3333], dtype=np.float16)
    rows = []
    for s in scales:
        for z in range(16):
            rows.append((s, z))
    oc = len(rows)
    codes = np.tile(np.arange(16, dtype=np.uint8), 8)[None, :].repeat(oc, 0)       # 128 columns, one group
    qweight = O.pack_int4_to_int32(codes.reshape(oc, 16, 8))
    zeros = np.full((oc, 8), 8, dtype=np.uint8)
    zeros[:, 0] = [z for _, z in rows]
    qzeros = O.pack_int4_to_int32(zeros.reshape(oc, 1, 8))
    sc = np.array([[s] for s, _ in rows], dtype=np.float16)
    got = ext().dequant(dev(qweight), dev(sc), dev(qzeros), 128, 128)
    want = O.dequant_full(qweight, qzeros, sc, 128, 128)
    np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), want.view(np.uint16))


# ---------------------------------------------------------------------------------------------- plain W4A16
@pytest.mark.parametrize("oc,ic", [(2048, 2048), (1024, 3072), (256, 8192), (40, 1152), (16, 128), (72, 136)])
@pytest.mark.parametrize("M", [1, 3, 8, 16, 32])
def test_plain_gemv_parity(oc, ic, M):
    rng = np.random.default_rng(oc * 7 + ic + M)
    lin = Linear(rng, oc, ic, bias=(oc == 40))
    x = rng.standard_normal((M, ic)).astype(np.float16)
    out = new_out(M, lin)
    g = make_group(dev(x), [lin], [out], kernel=K.KERNEL_GEMV)
    assert run_group(g) == 0
    assert_close(out, lin.oracle(x), tag=f"{oc}x{ic} M{M}")


def test_fp32_output_is_tighter():
    rng = np.random.default_rng(11)
    lin = Linear(rng, 512, 2048)
    x = rng.standard_normal((4, 2048)).astype(np.float16)
    out = new_out(4, lin, K.OUT_F32)
    g = make_group(dev(x), [lin], [out], out_dtype=K.OUT_F32, kernel=K.KERNEL_GEMV)
    assert run_group(g) == 0
    assert_close(out, lin.oracle(x), tol_abs=2e-3, tol_rel=2e-4)


@pytest.mark.parametrize("split_k", [2, 3, 8])
def test_split_k_matches_and_is_deterministic(split_k):
    rng = np.random.default_rng(split_k)
    lin = Linear(rng, 96, 4096, rank=32)
    R = (rng.standard_normal((32, 4096)) * 0.01).astype(np.float16)
    x = rng.standard_normal((5, 4096)).astype(np.float16)
    outs = []
    for _ in range(2):
        out = new_out(5, lin)
        r_buf = torch.zeros(5, 32, dtype=torch.float16, device="cuda")
        g = make_group(dev(x), [lin], [out], R_d=dev(R), r_buf=r_buf, r_mode=K.R_COMPUTE, split_k=split_k,
                       kernel=K.KERNEL_GEMV)
        assert run_group(g) == 0 and status_ok(g) == 0
        outs.append(out.cpu().numpy().copy())
    assert_close(torch.from_numpy(outs[0]), lin.oracle(x, R))
    np.testing.assert_array_equal(outs[0].view(np.uint16), outs[1].view(np.uint16))


@pytest.mark.parametrize("gs,ic", [(32, 256), (64, 1024), (8, 72)])
def test_other_group_sizes_take_the_generic_kernel(gs, ic):
    rng = np.random.default_rng(gs)
    lin = Linear(rng, 24, ic, gs, bias=True, rank=16)
    R = (rng.standard_normal((16, ic)) * 0.01).astype(np.float16)
    x = rng.standard_normal((3, ic)).astype(np.float16)
    out = new_out(3, lin)
    r_buf = torch.zeros(3, 16, dtype=torch.float16, device="cuda")
    g = make_group(dev(x), [lin], [out], R_d=dev(R), r_buf=r_buf, r_mode=K.R_COMPUTE, alpha=0.7)
    assert run_group(g) == 0
    assert_close(out, lin.oracle(x, R, alpha=0.7))


# ---------------------------------------------------------------------------------------------- corrected
@pytest.mark.parametrize("M", [1, 16])
@pytest.mark.parametrize("fused", [False, True])
def test_config1_qkv_group(M, fused):
    """OPT-1.3B-shaped QKV group: d = 2048, three 2048->2048 linears, g = 128, rank 64, checked per module.
    fused=False follows the wrapper protocol (q computes r, k and v load it); fused=True is one launch."""
    rng = np.random.default_rng(0)
    lins = [Linear(rng, 2048, 2048, rank=64) for _ in range(3)]
    R = (np.random.default_rng(1).standard_normal((64, 2048)) * 0.01).astype(np.float16)
    x = np.random.default_rng(2).standard_normal((M, 2048)).astype(np.float16)
    x_d, R_d = dev(x), dev(R)
    r_buf = torch.zeros(M, 64, dtype=torch.float16, device="cuda")
    outs = [new_out(M, l) for l in lins]
    if fused:
        g = make_group(x_d, lins, outs, R_d=R_d, r_buf=r_buf, r_mode=K.R_COMPUTE)
        assert run_group(g) == 0 and status_ok(g) == 0
    else:
        for i, (l, o) in enumerate(zip(lins, outs)):
            g = make_group(x_d, [l], [o], R_d=R_d, r_buf=r_buf, r_mode=K.R_COMPUTE if i == 0 else K.R_LOAD)
            assert run_group(g) == 0 and status_ok(g) == 0
    r_want = x.astype(np.float32) @ R.astype(np.float32).T
    assert np.abs(r_buf.float().cpu().numpy() - r_want).max() <= 2e-3
    for i, (l, o) in enumerate(zip(lins, outs)):
        assert_close(o, l.oracle(x, R), tag=f"member {i}")


@pytest.mark.parametrize("tag,d,rank,bias", [("qkv2048", 2048, 64, False), ("qkv1152b", 1152, 32, True)])
@pytest.mark.parametrize("M", [1, 16])
@pytest.mark.parametrize("alpha", [1.0, 0.5, 0.0])
def test_golden_forward_vectors(golden_forward, tag, d, rank, bias, M, alpha):
    """Inputs from the fixtures, outputs against what the reference's own wrapper produced (fp16 and fp32 runs)."""
    f = golden_forward
    x, R = f[f"{tag}.x{M}"], f[f"{tag}.R"]
    x_d, R_d = dev(x), dev(R)
    for od, odt in (("fp16", K.OUT_F16), ("fp32", K.OUT_F32)):
        r_buf = torch.zeros(M, rank, dtype=torch.float16, device="cuda")
        for i, n in enumerate(("q_proj", "k_proj", "v_proj")):
            lin = Linear.__new__(Linear)
            lin.oc, lin.ic, lin.gs = f[f"{tag}.{n}.qweight"].shape[0], d, 128
            lin.d_qweight, lin.d_qzeros, lin.d_scales = (dev(f[f"{tag}.{n}.qweight"]), dev(f[f"{tag}.{n}.qzeros"]),
                                                         dev(f[f"{tag}.{n}.scales"]))
            lin.d_bias = dev(f[f"{tag}.{n}.bias"]) if bias else None
            lin.d_L = dev(f[f"{tag}.{n}.L"])
            out = new_out(M, lin, odt)
            mode = K.R_NONE if alpha == 0.0 else (K.R_COMPUTE if i == 0 else K.R_LOAD)
            g = make_group(x_d, [lin], [out], R_d=R_d, r_buf=r_buf, r_mode=mode, alpha=alpha, out_dtype=odt)
            assert run_group(g) == 0
            assert_close(out, f[f"{tag}.y.M{M}.{od}.a{alpha}.{n}"].astype(np.float32), tag=f"{n} {od}")


@pytest.mark.parametrize("rank", [8, 16, 24, 40, 72, 264])
def test_ranks_that_are_not_multiples_of_32(rank):
    rng = np.random.default_rng(rank)
    lin = Linear(rng, 80, 1024, rank=rank, bias=True)
    R = (rng.standard_normal((rank, 1024)) * 0.01).astype(np.float16)
    x = rng.standard_normal((9, 1024)).astype(np.float16)
    out = new_out(9, lin)
    r_buf = torch.zeros(9, rank, dtype=torch.float16, device="cuda")
    g = make_group(dev(x), [lin], [out], R_d=dev(R), r_buf=r_buf, r_mode=K.R_COMPUTE)
    assert run_group(g) == 0 and status_ok(g) == 0
    assert_close(out, lin.oracle(x, R))


def test_mixed_group_members_alpha_and_missing_L():
    """gate/up style group where one member is uncorrected and alphas differ."""
    rng = np.random.default_rng(3)
    lins = [Linear(rng, 272, 1024, rank=128), Linear(rng, 48, 1024, rank=128, bias=True), Linear(rng, 160, 1024, rank=128)]
    R = (rng.standard_normal((128, 1024)) * 0.01).astype(np.float16)
    x = rng.standard_normal((7, 1024)).astype(np.float16)
    outs = [new_out(7, l) for l in lins]
    r_buf = torch.zeros(7, 128, dtype=torch.float16, device="cuda")
    g = make_group(dev(x), lins, outs, R_d=dev(R), r_buf=r_buf, r_mode=K.R_COMPUTE, alpha=[1.0, 0.25, 1.0],
                   use_L=[True, True, False])
    assert run_group(g) == 0 and status_ok(g) == 0
    assert_close(outs[0], lins[0].oracle(x, R))
    assert_close(outs[1], lins[1].oracle(x, R, alpha=0.25))
    assert_close(outs[2], lins[2].oracle(x, None))


def test_counters_rearm_over_many_launches():
    rng = np.random.default_rng(4)
    lin = Linear(rng, 1024, 3072, rank=64)
    R = (rng.standard_normal((64, 3072)) * 0.01).astype(np.float16)
    x = rng.standard_normal((2, 3072)).astype(np.float16)
    out = new_out(2, lin)
    r_buf = torch.zeros(2, 64, dtype=torch.float16, device="cuda")
    g = make_group(dev(x), [lin], [out], R_d=dev(R), r_buf=r_buf, r_mode=K.R_COMPUTE)
    e = ext()
    first = None
    for it in range(40):
        assert e.lib.glowq_w4a16_group_forward(g) == 0
        if it in (0, 39):
            torch.cuda.synchronize()
            cur = out.cpu().numpy().copy()
            first = cur if first is None else first
            np.testing.assert_array_equal(cur.view(np.uint16), first.view(np.uint16))
    assert status_ok(g) == 0
    head = g._keep[5][:16].view(torch.int32).cpu().numpy()
    assert (head[:4] == 0).all(), head          # ticket / done / exit / status all back to zero
    assert_close(out, lin.oracle(x, R))


@pytest.mark.parametrize("ocs,ic,rank,M,with_res", [([512, 128, 128], 1024, 64, 1, True), ([512, 128, 128], 1024, 64, 5, False),
                                                   ([256], 8192, 32, 2, True), ([3072, 1024, 1024], 3072, 64, 1, True)])
def test_fused_residual_rmsnorm_prologue(ocs, ic, rank, M, with_res):
    """The launch stages xn = w * fp16(rstd * fp16(x + residual)) instead of x (and hands h = x + residual back): every
    member's output and r against the oracle evaluated on the oracle's own xn; h bit for bit.  The long-K case runs
    K-sliced, where every slice needs the statistics of the whole row."""
    rng = np.random.default_rng(ic + M)
    lins = [Linear(rng, oc, ic, rank=rank) for oc in ocs]
    R = (rng.standard_normal((rank, ic)) * 0.01).astype(np.float16)
    x = rng.standard_normal((M, ic)).astype(np.float16)
    res = (rng.standard_normal((M, ic)) * 2).astype(np.float16) if with_res else None
    w = (1 + 0.2 * rng.standard_normal(ic)).astype(np.float16)
    xn, h = O.residual_rmsnorm_f16(x, res, w, 1e-5)
    outs = [new_out(M, l) for l in lins]
    r_buf = torch.zeros(M, rank, dtype=torch.float16, device="cuda")
    g = make_group(dev(x), lins, outs, R_d=dev(R), r_buf=r_buf, r_mode=K.R_COMPUTE)
    w_d, res_d = dev(w), (dev(res) if with_res else None)
    h_d = torch.zeros(M, ic, dtype=torch.float16, device="cuda")
    g.norm_weight, g.norm_eps, g.hidden_out = w_d.data_ptr(), 1e-5, h_d.data_ptr()
    g.residual = res_d.data_ptr() if with_res else None
    for _ in range(2):
        assert run_group(g) == 0 and status_ok(g) == 0
    np.testing.assert_array_equal(h_d.cpu().numpy().view(np.uint16), h.view(np.uint16))
    for l, o in zip(lins, outs):
        assert_close(o, l.oracle(xn, R), tag=f"norm {l.oc}x{l.ic} M={M}")
    r_want = xn.astype(np.float32) @ R.astype(np.float32).T
    assert np.abs(r_buf.float().cpu().numpy() - r_want).max() <= 6e-3
    # more than 8 tokens or the tensor-core kernel: refused, nothing runs
    g.kernel = K.KERNEL_GEMM
    assert ext().lib.glowq_w4a16_group_forward(g) == 8
    g.kernel, g.norm_weight = K.KERNEL_AUTO, None
    assert ext().lib.glowq_w4a16_group_forward(g) == 1          # residual / hidden_out without a norm weight



@pytest.mark.parametrize("M,ic,rank", [(9, 1152, 8), (16, 2048, 64), (40, 3200, 24), (64, 1024, 136), (65, 2176, 64),
                                       (128, 5120, 128), (129, 2048, 64)])
def test_r_for_few_tokens_and_the_group_gemm(M, ic, rank):
    """9..128 tokens take the tensor-core GEMM, with r = x R^T from the small stand-alone launch (one CTA per 16 rows
    of R x 1024 columns x 64 tokens, K slices added in order by the last CTA to arrive); 129 tokens take the K-sliced
    GEMM for r.  Ranks that are not multiples of 16, K that is not a multiple of 1024, token counts that do not fill
    the 64-token blocks; run twice on the same workspace (the arrival counters must be back at zero)."""
    rng = np.random.default_rng(40 + M)
    lins = [Linear(rng, oc, ic, rank=rank) for oc in (384, 200)]
    R = (np.random.default_rng(41).standard_normal((rank, ic)) * 0.01).astype(np.float16)
    x = np.random.default_rng(42).standard_normal((M, ic)).astype(np.float16)
    x_d, R_d = dev(x), dev(R)
    r_want = x.astype(np.float32) @ R.astype(np.float32).T
    g = None
    for rep in range(2):
        r_buf = torch.zeros(M, rank, dtype=torch.float16, device="cuda")
        outs = [new_out(M, l) for l in lins]
        g = make_group(x_d, lins, outs, R_d=R_d, r_buf=r_buf, r_mode=K.R_COMPUTE, ws=None if g is None else g._keep[-1])
        assert run_group(g) == 0 and status_ok(g) == 0
        assert np.abs(r_buf.float().cpu().numpy() - r_want).max() <= 2e-3, f"r, pass {rep}"
        for i, (l, o) in enumerate(zip(lins, outs)):
            assert_close(o, l.oracle(x, R), tag=f"member {i}, pass {rep}")

# ---------------------------------------------------------------------------------------------- tensor-core GEMM
@pytest.mark.parametrize("M,oc,ic,rank,alpha,bias", [
    (64, 256, 512, 0, 1.0, False), (128, 128, 128, 0, 1.0, False), (200, 136, 1152, 0, 1.0, True),
    (257, 384, 1024, 64, 1.0, True), (300, 320, 1024, 40, 0.5, False), (1024, 1024, 3072, 128, 1.0, False),
    (2048, 512, 5120, 256, 1.0, False), (70, 72, 136, 16, 2.0, True)])
def test_gemm_parity(M, oc, ic, rank, alpha, bias):
    rng = np.random.default_rng(M + oc + ic + rank)
    lin = Linear(rng, oc, ic, rank=rank, bias=bias)
    x = rng.standard_normal((M, ic)).astype(np.float16)
    R = (rng.standard_normal((max(rank, 8), ic)) * 0.01).astype(np.float16)
    for odt in (K.OUT_F16, K.OUT_F32):
        out = new_out(M, lin, odt)
        if rank:
            r_buf = torch.zeros(M, rank, dtype=torch.float16, device="cuda")
            g = make_group(dev(x), [lin], [out], R_d=dev(R), r_buf=r_buf, r_mode=K.R_COMPUTE, alpha=alpha,
                           kernel=K.KERNEL_GEMM, out_dtype=odt)
        else:
            g = make_group(dev(x), [lin], [out], kernel=K.KERNEL_GEMM, out_dtype=odt)
        assert run_group(g) == 0 and status_ok(g) == 0
        assert_close(out, lin.oracle(x, R if rank else None, alpha=alpha), tag=f"gemm {M}x{oc}x{ic} r{rank}")
        if rank:
            r_want = x.astype(np.float32) @ R.astype(np.float32).T
            assert np.abs(r_buf.float().cpu().numpy() - r_want).max() <= 4e-3


@pytest.mark.parametrize("M,oc,ic,rank,alpha", [(64, 256, 2048, 1024, 1.0), (64, 256, 2048, 1024, 0.5),
                                                (48, 384, 1024, 512, 1.0), (2560, 4096, 1024, 1024, 1.0)])
def test_gemm_k_slices_that_start_inside_the_correction_steps(M, oc, ic, rank, alpha):
    """Large rank against a short K: with the K steps of weights and correction cut into slices, some slices
    begin (or lie wholly) in the correction steps.  Their first MMA must overwrite the accumulator, and an
    accumulator a slice never touches must count as zero."""
    rng = np.random.default_rng(M + rank)
    lin = Linear(rng, oc, ic, rank=rank, bias=True)
    x = rng.standard_normal((M, ic)).astype(np.float16)
    R = (rng.standard_normal((rank, ic)) * 0.01).astype(np.float16)
    out = new_out(M, lin, K.OUT_F32)
    r_buf = torch.zeros(M, rank, dtype=torch.float16, device="cuda")
    g = make_group(dev(x), [lin], [out], R_d=dev(R), r_buf=r_buf, r_mode=K.R_COMPUTE, alpha=alpha,
                   kernel=K.KERNEL_GEMM, out_dtype=K.OUT_F32)
    for _ in range(2):
        out.fill_(float("nan"))
        assert run_group(g) == 0 and status_ok(g) == 0
        assert_close(out, lin.oracle(x, R, alpha=alpha), tag=f"gemm r{rank} ic{ic} M{M} alpha{alpha}")


def test_gemm_group_and_cache_modes():
    """q computes r (one r product for the group), k and v load it; also the fused three-member call."""
    rng = np.random.default_rng(12)
    lins = [Linear(rng, 512, 2048, rank=64), Linear(rng, 128, 2048, rank=64, bias=True), Linear(rng, 128, 2048, rank=64)]
    R = (rng.standard_normal((64, 2048)) * 0.01).astype(np.float16)
    x = rng.standard_normal((384, 2048)).astype(np.float16)
    x_d, R_d = dev(x), dev(R)
    for fused in (True, False):
        outs = [new_out(384, l) for l in lins]
        r_buf = torch.zeros(384, 64, dtype=torch.float16, device="cuda")
        if fused:
            g = make_group(x_d, lins, outs, R_d=R_d, r_buf=r_buf, r_mode=K.R_COMPUTE, kernel=K.KERNEL_GEMM)
            assert run_group(g) == 0 and status_ok(g) == 0
        else:
            for i, (l, o) in enumerate(zip(lins, outs)):
                g = make_group(x_d, [l], [o], R_d=R_d, r_buf=r_buf, r_mode=K.R_COMPUTE if i == 0 else K.R_LOAD,
                               kernel=K.KERNEL_GEMM)
                assert run_group(g) == 0 and status_ok(g) == 0
        for l, o in zip(lins, outs):
            assert_close(o, l.oracle(x, R))


def test_gemm_shared_memory_weight_tile_is_bit_exact():
    """One-hot activations read the dequantised weight back through the tensor-core path: y[m, oc] = W[oc, m]
    exactly (a single product with 1.0 per output), so the tile the MMA consumes is bit-identical to the reference
    dequantisation."""
    rng = np.random.default_rng(13)
    for oc, ic in ((256, 512), (136, 256)):
        lin = Linear(rng, oc, ic, w_std=0.05)
        x = np.eye(ic, dtype=np.float16)
        out = new_out(ic, lin)
        g = make_group(dev(x), [lin], [out], kernel=K.KERNEL_GEMM)
        assert run_group(g) == 0 and status_ok(g) == 0
        want = O.dequant_full(lin.qweight, lin.qzeros, lin.scales, ic, 128)
        np.testing.assert_array_equal(out.cpu().numpy().T.copy().view(np.uint16), want.view(np.uint16))


def test_gemv_and_gemm_agree_at_the_switch_over():
    rng = np.random.default_rng(14)
    lin = Linear(rng, 640, 3072, rank=64)
    R = (rng.standard_normal((64, 3072)) * 0.01).astype(np.float16)
    for M in (32, 33, 64):
        x = rng.standard_normal((M, 3072)).astype(np.float16)
        ys = []
        for kern in (K.KERNEL_GEMV, K.KERNEL_GEMM, K.KERNEL_AUTO):
            out = new_out(M, lin, K.OUT_F32)
            r_buf = torch.zeros(M, 64, dtype=torch.float16, device="cuda")
            g = make_group(dev(x), [lin], [out], R_d=dev(R), r_buf=r_buf, r_mode=K.R_COMPUTE, kernel=kern,
                           out_dtype=K.OUT_F32)
            assert run_group(g) == 0 and status_ok(g) == 0
            ys.append(out.cpu().numpy())
            assert_close(out, lin.oracle(x, R), tol_abs=4e-3, tol_rel=3e-4)
        assert np.abs(ys[0] - ys[1]).max() <= 4e-3


# ---------------------------------------------------------------------------------------------- full-size shapes
LLAMA32_3B = dict(hidden=3072, inter=8192, kv=1024, rank=64)


@pytest.mark.parametrize("M", [1, 8, 32])
def test_llama32_3b_layer_shapes(M):
    """All seven linears of one Llama-3.2-3B-shaped layer at full size: qkv and gate/up as fused groups,
    o_proj and down_proj solo, against the C oracle."""
    c = LLAMA32_3B
    rng = np.random.default_rng(100 + M)
    h, it, kv, r = c["hidden"], c["inter"], c["kv"], c["rank"]
    x = rng.standard_normal((M, h)).astype(np.float16)
    xi = rng.standard_normal((M, it)).astype(np.float16)
    for members, inp, ic in (([h, kv, kv], x, h), ([h], x, h), ([it, it], x, h), ([h], xi, it)):
        lins = [Linear(rng, oc, ic, rank=r) for oc in members]
        R = (rng.standard_normal((r, ic)) * 0.01).astype(np.float16)
        outs = [new_out(M, l) for l in lins]
        r_buf = torch.zeros(M, r, dtype=torch.float16, device="cuda")
        g = make_group(dev(inp), lins, outs, R_d=dev(R), r_buf=r_buf, r_mode=K.R_COMPUTE)
        assert run_group(g) == 0 and status_ok(g) == 0
        for l, o in zip(lins, outs):
            assert_close(o, l.oracle(inp, R), tag=f"{l.oc}x{l.ic}")


def test_correction_term_is_linear_in_alpha():
    """Size-independent property at a full-size shape: y(alpha) - y(0) scales with alpha."""
    rng = np.random.default_rng(9)
    lin = Linear(rng, 5120, 5120, rank=256)
    R = (rng.standard_normal((256, 5120)) * 0.01).astype(np.float16)
    x = rng.standard_normal((4, 5120)).astype(np.float16)
    x_d, R_d = dev(x), dev(R)
    ys = {}
    for a in (0.0, 1.0, 2.0):
        out = new_out(4, lin, K.OUT_F32)
        r_buf = torch.zeros(4, 256, dtype=torch.float16, device="cuda")
        g = make_group(x_d, [lin], [out], R_d=R_d, r_buf=r_buf, r_mode=K.R_COMPUTE, alpha=a, out_dtype=K.OUT_F32)
        assert run_group(g) == 0
        ys[a] = out.cpu().numpy().astype(np.float64)
    d1, d2 = ys[1.0] - ys[0.0], ys[2.0] - ys[0.0]
    assert np.abs(d2 - 2 * d1).max() <= 1e-4
    corr = (x.astype(np.float32) @ R.astype(np.float32).T) @ lin.L.astype(np.float32).T
    assert np.abs(d1 - corr).max() <= 2e-3


# ---------------------------------------------------------------------------------------------- boundary behaviour
def test_error_codes_and_empty_input():
    rng = np.random.default_rng(5)
    lin = Linear(rng, 32, 256)
    x_d = dev(rng.standard_normal((2, 256)).astype(np.float16))
    out = new_out(2, lin)
    e = ext()
    g = make_group(x_d, [lin], [out])
    g.group_size = 12
    assert run_group(g) == 2
    g = make_group(x_d, [lin], [out])
    g.members[0].qweight = None
    assert run_group(g) == 1
    g = make_group(x_d, [lin], [out])
    g.members[0].weight_stride_i32 = 8
    assert run_group(g) == 3
    g = make_group(x_d, [lin], [out])
    g.workspace_bytes = 64
    assert run_group(g) == 4
    g = make_group(x_d, [lin], [out], r_mode=K.R_NONE)
    g.r_mode, g.rank = K.R_COMPUTE, 0
    assert run_group(g) == 1
    g = make_group(x_d[:0], [lin], [out[:0]])
    assert run_group(g) == 0                                   # M = 0: nothing to do
    with pytest.raises(RuntimeError, match="multiple of 8"):
        e.w4a16_gemv_forward_cuda(x_d, lin.d_qweight, lin.d_scales, lin.d_qzeros, 12)
    with pytest.raises(RuntimeError, match="fp16"):
        e.w4a16_gemv_forward_cuda(x_d.float(), lin.d_qweight, lin.d_scales, lin.d_qzeros, 128)


def test_reference_named_entry_points():
    rng = np.random.default_rng(6)
    lin = Linear(rng, 640, 2048)
    e = ext()
    for M in (1, 16, 48):
        x = rng.standard_normal((M, 2048)).astype(np.float16)
        want = lin.oracle(x)
        for fn in (e.w4a16_gemv_forward_cuda, e.gemv_w4a16_asym):
            y = fn(dev(x), lin.d_qweight, lin.d_scales, lin.d_qzeros, 128)
            assert y.dtype == torch.float16 and tuple(y.shape) == (M, 640)
            assert_close(y, want)
        y = e.w4a16_gemm_forward_cuda(dev(x), lin.d_qweight, lin.d_scales, lin.d_qzeros, 128, 1)
        assert_close(y, want)


def test_host_buffer_entry_point():
    rng = np.random.default_rng(8)
    lins = [Linear(rng, 320, 1024, rank=32), Linear(rng, 64, 1024, rank=32)]
    R = (rng.standard_normal((32, 1024)) * 0.01).astype(np.float16)
    x = rng.standard_normal((3, 1024)).astype(np.float16)
    x_host = torch.from_numpy(x).pin_memory()
    x_d = torch.zeros(3, 1024, dtype=torch.float16, device="cuda")
    outs = [new_out(3, l) for l in lins]
    outs_host = [torch.zeros(3, l.oc, dtype=torch.float16).pin_memory() for l in lins]
    r_buf = torch.zeros(3, 32, dtype=torch.float16, device="cuda")
    g = make_group(x_d, lins, outs, R_d=dev(R), r_buf=r_buf, r_mode=K.R_COMPUTE)
    ptrs = (ctypes.c_void_p * 2)(*[o.data_ptr() for o in outs_host])
    assert ext().lib.glowq_w4a16_group_forward_host(g, x_host.data_ptr(), ptrs) == 0
    for l, o in zip(lins, outs_host):
        assert_close(o, l.oracle(x, R))


# ---------------------------------------------------------------------------------------------- Python surface
@pytest.mark.parametrize("fuse", ["1", "0"])
def test_toy_model_through_wrappers_matches_reference(golden_toy, monkeypatch, fuse):
    """convert -> patch -> call in HF order on the GPU; outputs vs what the reference modules produced on CPU.
    fuse = 1: the patcher's group launchers issue one library call per q/k/v and gate/up group (k, v and up are
    served from the producer's launch); fuse = 0: one call per module (the wrapper protocol)."""
    monkeypatch.setenv("W4A16_KERNEL_OUT_DTYPE", "fp16")
    monkeypatch.setenv("GLOWQ_FUSE_GROUPS", fuse)
    from toy_model import ToyDecoder, make_artifacts
    import glowq_b200 as G
    from glowq_b200.cuda_w4a16.linear import CudaW4A16Linear
    model = G.convert_to_cuda_w4a16(ToyDecoder(), 128)
    shared, bmap = make_artifacts(model)
    model = model.cuda()
    G.patch_svd_correction_wrappers(model, shared, bmap, 1.0)
    launches = []
    real_launch = CudaW4A16Linear.launch
    monkeypatch.setattr(CudaW4A16Linear, "launch", lambda self, *a, **k: (launches.append(1), real_launch(self, *a, **k))[1])
    q0 = model.proj(0, "self_attn.q_proj")
    assert (q0.group_launcher is not None) == (fuse == "1")
    if fuse == "1":
        assert [w.role for w in q0.group_launcher.members] == ["q", "k", "v"]
        assert model.proj(0, "self_attn.k_proj").group_launcher is q0.group_launcher
        assert q0.group_launcher.next_launcher is model.proj(0, "self_attn.o_proj").group_launcher
    for M in (1, 5):
        x, xi = dev(golden_toy[f"x{M}"]), dev(golden_toy[f"xi{M}"])
        for li in range(2):
            for p in ToyDecoder.PROJ:
                y = model.proj(li, p)(xi if p.endswith("down_proj") else x)
                assert y.dtype == torch.float16
                assert_close(y, golden_toy[f"y{M}.{li}.{p}"].astype(np.float32), tag=f"{li}.{p}")
    # fused: every call went through a group launcher; per module: 7 launches per layer and token count
    assert len(launches) == (0 if fuse == "1" else 2 * 2 * 7)
    # a consumer that is called with ANOTHER tensor than its producer saw computes for itself
    x = dev(golden_toy["x5"])
    model.proj(0, "self_attn.q_proj")(x)
    other = (x * 0.5).contiguous()
    y = model.proj(0, "self_attn.k_proj")(other)
    assert_close(y * 2, golden_toy["y5.0.self_attn.k_proj"].astype(np.float32), tol_abs=4e-2, tol_rel=2e-3, tag="miss")
    # 3-D input keeps its leading dims; alpha 0 equals the bare module
    w = model.proj(0, "self_attn.q_proj")
    x3 = torch.randn(2, 3, 256, device="cuda", dtype=torch.float16)
    assert tuple(w(x3).shape) == (2, 3, 256)
    for name in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"):
        model.proj(0, name).alpha_svd = 0.0
    torch.testing.assert_close(w(x3), w.inner(x3))
    k = model.proj(0, "self_attn.k_proj")
    torch.testing.assert_close(k(x3), k.inner(x3))       # nothing kept from an earlier call is served
    # alpha 0 on one member only: it gets the bare product, the others keep their correction
    model.proj(0, "self_attn.q_proj").alpha_svd = 1.0
    y_q = w(x3)
    torch.testing.assert_close(k(x3), k.inner(x3), rtol=2e-3, atol=2e-3)
    assert float((y_q - w.inner(x3)).abs().max()) > 0


@pytest.mark.gpu
def test_gemm_with_a_sliced_last_wave():
    """160 tiles of 256 x 256 on 148 SMs: one whole wave, and a last wave of 12 tiles that is cut into K slices whose
    fp32 partial tiles are added by the slot-sum kernel (bias and correction included)."""
    M, oc, ic, rank = 2560, 4096, 1024, 64
    rng = np.random.default_rng(7)
    lin = Linear(rng, oc, ic, rank=rank, bias=True)
    x = rng.standard_normal((M, ic)).astype(np.float16)
    R = (rng.standard_normal((rank, ic)) * 0.01).astype(np.float16)
    for r_mode in (K.R_NONE, K.R_COMPUTE):
        out = new_out(M, lin)
        if r_mode == K.R_NONE:
            g = make_group(dev(x), [lin], [out], kernel=K.KERNEL_GEMM)
        else:
            r_buf = torch.zeros(M, rank, dtype=torch.float16, device="cuda")
            g = make_group(dev(x), [lin], [out], R_d=dev(R), r_buf=r_buf, r_mode=r_mode, alpha=1.0, kernel=K.KERNEL_GEMM)
        for _ in range(2):   # the second call reuses the slots
            assert run_group(g) == 0 and status_ok(g) == 0
        assert_close(out, lin.oracle(x, R if r_mode != K.R_NONE else None, alpha=1.0), tag="sliced last wave")


@pytest.mark.gpu
def test_cta_pair_variant_in_subprocess():
    """The two-CTA (cta_group::2) GEMM variant (above 128 tokens) and the swapped-operand variant (up to 128 tokens)
    are opt-in through environment variables that the library reads once, so they are exercised in a child
    interpreter: the GEMM parity tests must pass with both forced on."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, GLOWQ_GEMM_PAIR="1", GLOWQ_GEMM_SWAP="1")
    here = os.path.dirname(os.path.abspath(__file__))
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(here, "test_gpu_parity.py"), "-q", "-x", "-m", "gpu",
                        "-k", "gemm_parity or gemm_group or shared_memory_weight_tile", "-p", "no:cacheprovider"],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert " passed" in r.stdout
