"""The scratch-free entry point glowq_w4a16_gemv_forward_static against glowq_w4a16_gemv_forward.

Some callers can neither allocate device memory for us nor own a workspace (a plug-in that is only ever handed
input and output pointers, a serving loop with a frozen memory plan), so this variant keeps its scratch in an
array inside the library image.  It must give exactly what the workspace-taking entry point gives, call after
call, because all calls share that one array.  Collected last on purpose: a failure here cannot hide another test."""
import numpy as np
import pytest
import torch

from glowq_b200.cuda_w4a16 import kernels as K
from gpu_helpers import Linear, assert_close, dev, ext

pytestmark = pytest.mark.gpu


def _both(lin, x_d, M):
    e = ext()
    stream = torch.cuda.current_stream().cuda_stream
    want = e.w4a16_gemv_forward_cuda(x_d, lin.d_qweight, lin.d_scales, lin.d_qzeros, lin.gs)
    got = torch.full((M, lin.oc), float("nan"), dtype=torch.float16, device="cuda")
    rc = e.lib.glowq_w4a16_gemv_forward_static(x_d.data_ptr(), lin.d_qweight.data_ptr(), lin.d_scales.data_ptr(),
                                               lin.d_qzeros.data_ptr(), got.data_ptr(), M, lin.ic, lin.oc, lin.gs,
                                               lin.d_qweight.stride(0), lin.d_qzeros.stride(0), lin.d_scales.stride(0),
                                               stream)
    torch.cuda.synchronize()
    return rc, got, want


@pytest.mark.parametrize("oc,ic,M", [(1024, 3072, 1), (96, 8192, 5), (3072, 2048, 16)])
def test_static_scratch_matches_workspace_entry_point_twice_in_a_row(oc, ic, M):
    rng = np.random.default_rng(oc + M)
    lin = Linear(rng, oc, ic)
    for call in range(2):                      # second call reuses whatever the first left in the shared array
        x = rng.standard_normal((M, ic)).astype(np.float16)
        rc, got, want = _both(lin, dev(x), M)
        assert rc == 0, rc
        # same kernel, same plan, same summation order: identical bits, and inside the oracle tolerances
        np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), want.cpu().numpy().view(np.uint16))
        assert_close(got, lin.oracle(x), tag=f"call {call}")
    # callers of this entry point own no workspace: NULL addresses the built-in scratch's status word
    assert ext().lib.glowq_w4a16_read_status(None, torch.cuda.current_stream().cuda_stream) == 0


def test_static_scratch_rejects_what_does_not_fit():
    """A launch plan whose partial sums exceed the built-in array is refused with a clear status, nothing runs."""
    e = ext()
    rng = np.random.default_rng(1)
    lin = Linear(rng, 32, 128)
    x_d = dev(rng.standard_normal((1, 128)).astype(np.float16))
    out = torch.zeros(1, 32, dtype=torch.float16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # pretend-huge output dimension: only the plan is evaluated before the size check
    rc = e.lib.glowq_w4a16_gemv_forward_static(x_d.data_ptr(), lin.d_qweight.data_ptr(), lin.d_scales.data_ptr(),
                                               lin.d_qzeros.data_ptr(), out.data_ptr(), 1, 128, 1 << 26, 128,
                                               lin.d_qweight.stride(0), lin.d_qzeros.stride(0), lin.d_scales.stride(0),
                                               stream)
    assert rc == 9 and b"maximum" in e.lib.glowq_w4a16_strerror(rc)
    rc = e.lib.glowq_w4a16_gemv_forward_static(x_d.data_ptr(), lin.d_qweight.data_ptr(), lin.d_scales.data_ptr(),
                                               lin.d_qzeros.data_ptr(), out.data_ptr(), 1, 128, 32, 12,
                                               lin.d_qweight.stride(0), lin.d_qzeros.stride(0), lin.d_scales.stride(0),
                                               stream)
    assert rc == 2
