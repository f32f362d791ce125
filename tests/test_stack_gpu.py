"""The benchmark workload (LinearStack) computes what it claims: every output of one token step of a one-layer
stack against the CPU oracle, for the fused-group and the per-module launch plans, decode and prefill sizes."""
import numpy as np
import pytest
import torch

import c_oracle as C
from glowq_b200.cuda_w4a16 import kernels as K
from glowq_b200.stack import SHAPES, LinearStack, StackShape
from gpu_helpers import assert_close

pytestmark = pytest.mark.gpu


def _oracle(member, x, R, use_corr):
    return C.corrected_forward(x, member.qweight.cpu().numpy(), member.scales.cpu().numpy(), member.qzeros.cpu().numpy(),
                               128, bias=None if member.bias is None else member.bias.cpu().numpy(),
                               R=R.cpu().numpy() if use_corr else None, L=member.L.cpu().numpy() if use_corr else None)


@pytest.mark.parametrize("M", [1, 8, 96])
@pytest.mark.parametrize("fuse", [True, False])
def test_one_layer_step_matches_oracle(M, fuse):
    shape = StackShape("mini", 1, 1024, 2816, 8, 2, 128, 64, qkv_bias=True)
    mask = {"layer0_qkv", "model.layers.0.mlp.down_proj"}            # GlowQ-S style: two of the four groups corrected
    stack = LinearStack(shape, "cuda", seed=3, enabled_groups=mask)
    plan = stack.plan(M, corrected=True, fuse_groups=fuse)
    stack.step(plan)
    torch.cuda.synchronize()
    stack.check_status(plan)
    outs = [item for item in plan["keep"] if isinstance(item, list) and item and isinstance(item[0], torch.Tensor)
            and item[0].dim() == 2 and item[0].dtype == torch.float16 and item[0].size(0) == M]
    assert len(outs) == len(stack.groups)
    for g, o_list in zip(stack.groups, outs):
        x = plan["inputs"][g.input_name].cpu().numpy()
        for m, o in zip(g.members, o_list):
            assert_close(o, _oracle(m, x, g.R, g.enabled), tag=f"{g.key} M={M}")
    assert stack.algorithmic_bytes(M) > stack.algorithmic_bytes(M, corrected=False)


def test_named_shapes_cover_the_baseline_configs():
    assert SHAPES["llama-3.2-3b"].q_out == 3072 and SHAPES["llama-3.2-3b"].kv_out == 1024
    assert SHAPES["qwen2.5-7b"].qkv_bias and SHAPES["qwen2.5-7b"].inter == 18944
    assert SHAPES["llama-2-13b"].rank == 128 and SHAPES["qwen3-14b"].rank == 256
    assert LinearStack._row_shard_cols(13824, 8, 0) == 1792 and LinearStack._row_shard_cols(13824, 8, 7) == 1664
