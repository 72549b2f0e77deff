"""GPU test of lyraq_w4a4_forward_static, the W4A4 forward for hosts that cannot allocate device memory.

The entry point keeps its scratch (packed int4 activation + group scales) in a fixed array inside the library, so a
caller passes inputs and outputs only.  It must give exactly what lyraq_w4a4_forward gives with a caller-owned
workspace, on the first call and again on a second call that finds the previous call's bytes in the array, and it must
refuse a problem that does not fit.  The file name sorts last on purpose: a run that stops at the first failure has
then already been through every other test.  The test stands alone in a fresh process as well.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(m, k, n, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g).bfloat16().cuda()
    w = (torch.randn(n, k, generator=g) * 0.02).bfloat16().cuda()
    smooth = (0.5 + torch.rand(k, generator=g)).float().cuda()
    bias = (torch.randn(n, generator=g) * 0.1).bfloat16().cuda()
    return x, w, smooth, bias


def test_static_scratch_forward_matches_workspace_forward_twice_in_a_row():
    from lyradiff_b200 import _lib, layers, ops

    L = _lib.lib()
    cap = L.lyraq_static_scratch_bytes()       # also the start-up warm-up: resolves the array on this device
    assert cap == 16 << 20
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second one finds the first one's bytes in the array
    for call, (m, k, n) in enumerate([(300, 512, 264), (130, 3072, 392)]):
        x, w, smooth, bias = _case(m, k, n, seed=40 + call)
        lin = layers.W4A4Gemm.from_float(w, smooth=smooth, bias=bias)
        want = lin.forward(x)                         # caller-owned workspace
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        st = L.lyraq_w4a4_forward_static(got.data_ptr(), x.data_ptr(), ops.BF16, smooth.data_ptr(), lin.qweight.data_ptr(),
                                         lin.w_scale.data_ptr(), ops._dt(lin.w_scale), bias.data_ptr(), None, ops.EPI_NONE,
                                         m, n, k, stream)
        assert st == 0, L.lyraq_status_string(st)
        torch.cuda.synchronize()
        # same kernels, same arithmetic: the tolerance the W4A4 tests use is bit equality
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), "call %d differs" % call
        # and directly against the CPU oracle, as the other W4A4 tests do (exact int32 group sums, fp32 rescale in group order)
        from oracle import gemm as ogemm
        from oracle import quant as oquant
        _, sa, qa = oquant.int4_quant_g64(x.cpu(), smooth.cpu())
        ref = ogemm.w4a4_gemm(qa, oquant.unpack_int4(lin.qweight.cpu()), sa, lin.w_scale.cpu(), bias=bias.cpu())
        assert torch.equal(got.cpu().view(torch.int16), ref.view(torch.int16)), "call %d differs from the oracle" % call
    status, detail = ops.last_status()
    assert status == 0, detail


def test_static_scratch_forward_refuses_what_does_not_fit():
    from lyradiff_b200 import _lib

    L = _lib.lib()
    # 65536 x 4096 needs 128 MiB of packed activation: far beyond the 16 MiB array -> refused before any launch
    p = 0x10000
    st = L.lyraq_w4a4_forward_static(p, p, 1, None, p, p, 2, None, None, 0, 65536, 256, 4096, None)
    assert st == 5  # LYRAQ_ERR_WORKSPACE
    assert L.lyraq_w4a4_forward_static(p, p, 1, None, p, p, 2, None, None, 0, 0, 256, 4096, None) == 0  # empty problem
