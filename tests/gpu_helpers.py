"""Shared plumbing of the GPU parity tests: seeded cases from the oracle, device upload, C-ABI calls."""
import ctypes

import numpy as np
import torch

import c_oracle as C
import glowq_oracle as O
from glowq_b200.cuda_w4a16 import kernels as K

TOL_ABS, TOL_REL = 2e-2, 1e-3      # max-abs / mean-rel against the fp32 oracle (the stated tolerances)


def ext():
    return K.load_w4a16_extension()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


class Linear:
    """One quantised linear: numpy originals + device copies."""

    def __init__(self, rng, oc, ic, gs=128, bias=False, rank=0, w_std=0.02, quantize=True):
        self.oc, self.ic, self.gs = oc, ic, gs
        if quantize:
            w = (rng.standard_normal((oc, ic)) * w_std).astype(np.float16)
            self.qweight, self.qzeros, self.scales, self.icp = O.quantize_per_group_w4(w, gs)
        else:
            # codes, zero-points and scales drawn directly, in the ranges RTN gives N(0, w_std) weights (no quantiser
            # pass: seconds instead of tens of seconds for the largest shapes); unused zero nibbles hold 8 as the
            # packer leaves them
            assert ic % gs == 0
            G = ic // gs
            self.icp = ic
            self.qweight = rng.integers(-2**31, 2**31, size=(oc, ic // 8), dtype=np.int64).astype(np.int32)
            z = rng.integers(0, 16, size=(oc, (G + 7) // 8 * 8), dtype=np.int64)
            z[:, G:] = 8
            zw = np.zeros((oc, (G + 7) // 8), dtype=np.int64)
            for j in range(8):
                zw |= z[:, j::8] << (4 * j)
            self.qzeros = (zw & 0xFFFFFFFF).astype(np.uint32).view(np.int32)
            self.scales = rng.uniform(0.3 * w_std, 0.55 * w_std, size=(oc, G)).astype(np.float16)
        self.bias = (rng.standard_normal(oc) * 0.1).astype(np.float16) if bias else None
        self.L = (rng.standard_normal((oc, rank)) * 0.01).astype(np.float16) if rank else None
        self.d_qweight, self.d_qzeros, self.d_scales = dev(self.qweight), dev(self.qzeros), dev(self.scales)
        self.d_bias = dev(self.bias) if bias else None
        self.d_L = dev(self.L) if rank else None

    def oracle(self, x, R=None, alpha=1.0, use_L=True):
        L = self.L if (use_L and R is not None) else None
        return C.corrected_forward(x, self.qweight, self.scales, self.qzeros, self.gs, bias=self.bias,
                                   R=R if L is not None else None, L=L, alpha=alpha)


def make_group(x_d, lins, outs, *, R_d=None, r_buf=None, r_mode=K.R_NONE, alpha=1.0, out_dtype=K.OUT_F16,
               kernel=K.KERNEL_AUTO, split_k=0, ws=None, use_L=None, stream=None):
    e = ext()
    g = K.Group()
    M, IC = x_d.shape
    g.x, g.M, g.IC, g.x_stride = x_d.data_ptr(), M, IC, x_d.stride(0)
    g.group_size = lins[0].gs
    g.r_mode = r_mode
    g.out_dtype, g.kernel, g.split_k = out_dtype, kernel, split_k
    rank = 0
    if r_mode != K.R_NONE:
        rank = r_buf.size(1)
        g.rank = rank
        g.r_buf = r_buf.data_ptr()
        if R_d is not None:
            g.R, g.R_stride = R_d.data_ptr(), R_d.stride(0)
    g.n_members = len(lins)
    alphas = alpha if isinstance(alpha, (list, tuple)) else [alpha] * len(lins)
    use_L = use_L if use_L is not None else [True] * len(lins)
    for i, (lin, out) in enumerate(zip(lins, outs)):
        m = g.members[i]
        m.qweight, m.scales, m.qzeros = lin.d_qweight.data_ptr(), lin.d_scales.data_ptr(), lin.d_qzeros.data_ptr()
        m.bias = lin.d_bias.data_ptr() if lin.d_bias is not None else None
        if r_mode != K.R_NONE and lin.d_L is not None and use_L[i]:
            m.L, m.L_stride = lin.d_L.data_ptr(), lin.d_L.stride(0)
        m.out, m.out_stride, m.OC = out.data_ptr(), out.stride(0), lin.oc
        m.weight_stride_i32, m.zero_stride_i32, m.scale_stride = (lin.d_qweight.stride(0), lin.d_qzeros.stride(0),
                                                                  lin.d_scales.stride(0))
        m.alpha = float(alphas[i])
    if ws is None:
        need = e.workspace_bytes(max(M, 1), IC, sum(l.oc for l in lins), rank, len(lins))
        ws = torch.zeros(max(need, 256) + (64 << 20 if split_k else 0), dtype=torch.uint8, device="cuda")
    g.workspace, g.workspace_bytes = ws.data_ptr(), ws.numel()
    g.stream = stream if stream is not None else torch.cuda.current_stream().cuda_stream
    g._keep = (x_d, lins, outs, R_d, r_buf, ws)
    return g


def run_group(g):
    e = ext()
    rc = e.lib.glowq_w4a16_group_forward(g)
    torch.cuda.synchronize()
    return rc


def status_ok(g):
    return ext().lib.glowq_w4a16_read_status(g.workspace, g.stream)


def new_out(M, lin, out_dtype=K.OUT_F16):
    return torch.full((M, lin.oc), float("nan"), dtype=torch.float16 if out_dtype == K.OUT_F16 else torch.float32,
                      device="cuda")


def assert_close(y_d, want, tol_abs=TOL_ABS, tol_rel=TOL_REL, tag=""):
    got = y_d.float().cpu().numpy()
    assert np.isfinite(got).all(), f"{tag}: non-finite output"
    ma, mr = O.parity_errors(got, want)
    assert ma <= tol_abs and mr <= tol_rel, f"{tag}: max-abs {ma:.3e} mean-rel {mr:.3e}"
    return ma, mr
