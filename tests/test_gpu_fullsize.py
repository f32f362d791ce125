"""Full-size parity: one decoder layer each of the Qwen2.5-7B, Llama-2-13B and Qwen3-14B shapes through both kernels.

These are the shapes whose sizes exercise what the small cases cannot: 28 and 148 quantisation groups (zero-point
words with pad nibbles, rows whose group count is not a multiple of the pipeline stage), q/k/v bias, 108 and 136
groups behind a K-sliced down_proj, rank 128 and 256.  Every output is compared with the C oracle inside the stated
tolerances; for large token counts the oracle is evaluated on a seeded sample of output rows of each member (the GPU
still computes everything), and the packed weights are drawn directly instead of quantised, which keeps the file to
about a minute of CPU time."""
import numpy as np
import pytest
import torch

import c_oracle as C
from glowq_b200.cuda_w4a16 import kernels as K
from gpu_helpers import Linear, assert_close, dev, make_group, new_out, run_group, status_ok

pytestmark = pytest.mark.gpu

CONFIGS = {
    # name: hidden, intermediate, q rows, kv rows, rank, q/k/v bias
    "qwen2.5-7b": dict(h=3584, inter=18944, q=3584, kv=512, rank=128, bias=True),
    "llama-2-13b": dict(h=5120, inter=13824, q=5120, kv=5120, rank=128, bias=False),
    "qwen3-14b": dict(h=5120, inter=17408, q=5120, kv=1024, rank=256, bias=False),
}
ORACLE_MAC_BUDGET = 3e9      # multiply-adds of the CPU oracle per member before rows are sampled


class Layer:
    def __init__(self, name):
        c = CONFIGS[name]
        rng = np.random.default_rng(500 + list(CONFIGS).index(name))
        r = c["rank"]
        self.rank = r
        self.groups = []      # (input width, members, R)
        for ocs, ic, bias in (([c["q"], c["kv"], c["kv"]], c["h"], c["bias"]), ([c["h"]], c["q"], False),
                              ([c["inter"], c["inter"]], c["h"], False), ([c["h"]], c["inter"], False)):
            lins = [Linear(rng, oc, ic, rank=r, bias=bias, quantize=False) for oc in ocs]
            R = (rng.standard_normal((r, ic)) * 0.01).astype(np.float16)
            self.groups.append((ic, lins, R, dev(R)))
        self.rng = rng


@pytest.fixture(scope="module", params=list(CONFIGS))
def layer(request):
    return request.param, Layer(request.param)


def _oracle_rows(lin, x, R, rows):
    return C.corrected_forward(x, lin.qweight[rows], lin.scales[rows], lin.qzeros[rows], lin.gs,
                               bias=None if lin.bias is None else lin.bias[rows], R=R, L=lin.L[rows], alpha=1.0)


@pytest.mark.parametrize("M", [1, 16, 64, 2048])
def test_one_layer_of_each_config(layer, M):
    name, lay = layer
    rng = np.random.default_rng(M)
    for ic, lins, R, R_d in lay.groups:
        x = rng.standard_normal((M, ic)).astype(np.float16)
        outs = [new_out(M, l) for l in lins]
        r_buf = torch.zeros(M, lay.rank, dtype=torch.float16, device="cuda")
        g = make_group(dev(x), lins, outs, R_d=R_d, r_buf=r_buf, r_mode=K.R_COMPUTE)   # automatic kernel choice
        assert run_group(g) == 0 and status_ok(g) == 0, (name, ic, M)
        for l, o in zip(lins, outs):
            if M * l.oc * l.ic <= ORACLE_MAC_BUDGET:
                rows = np.arange(l.oc)
            else:
                n = max(64, int(ORACLE_MAC_BUDGET // (M * l.ic)) // 32 * 32)
                rows = np.sort(rng.choice(l.oc, size=min(n, l.oc), replace=False))
            want = _oracle_rows(l, x, R, rows)
            got = o[:, torch.from_numpy(rows).cuda()]
            assert_close(got, want, tag=f"{name} {l.oc}x{l.ic} M={M}")
        r_want = x.astype(np.float32) @ R.astype(np.float32).T
        assert np.abs(r_buf.float().cpu().numpy() - r_want).max() <= 6e-3, (name, ic, M)


@pytest.mark.parametrize("M,kernel", [(8, K.KERNEL_GEMM), (16, K.KERNEL_GEMV)])
def test_both_kernels_on_the_ragged_group_counts(layer, M, kernel):
    """The kernel the automatic choice would NOT take at this token count, on the q/k/v group (bias, 28 / 40 groups)
    and on down_proj (148 / 108 / 136 groups)."""
    name, lay = layer
    rng = np.random.default_rng(77 + M)
    for gi in (0, 3):
        ic, lins, R, R_d = lay.groups[gi]
        x = rng.standard_normal((M, ic)).astype(np.float16)
        outs = [new_out(M, l) for l in lins]
        r_buf = torch.zeros(M, lay.rank, dtype=torch.float16, device="cuda")
        g = make_group(dev(x), lins, outs, R_d=R_d, r_buf=r_buf, r_mode=K.R_COMPUTE, kernel=kernel)
        assert run_group(g) == 0 and status_ok(g) == 0, (name, ic, M)
        for l, o in zip(lins, outs):
            assert_close(o, l.oracle(x, R), tag=f"{name} {l.oc}x{l.ic} M={M} kernel={kernel}")
