"""GPU parity tests of the INT8 W8A8 tcgen05 GEMM against the CPU oracle, through the C ABI.
Integer accumulators are compared bit for bit; the fp16/bf16 outputs too, because the epilogue
follows the oracle's rounding sequence exactly (T(T(acc*scale)+bias))."""

import pytest
import torch

from oracle import gemm, quant, workloads
from tests.util import assert_bit_equal, check_status, cu

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from lyradiff_b200 import ops as _ops
    return _ops


@pytest.fixture(params=[0, 2561, 1281, 2562], ids=["auto", "1cta_n256", "1cta_n128", "pair_n256"])
def tile(request):
    """Runs a test once per tile configuration of the dense GEMM (automatic choice, and each kernel variant forced)."""
    from lyradiff_b200 import _lib
    assert _lib.lib().lyraq_debug_force_gemm_tile(request.param) == 0
    yield request.param
    _lib.lib().lyraq_debug_force_gemm_tile(0)


def _rand_int8(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(-128, 128, (m, k), generator=g, dtype=torch.int8)
    b = torch.randint(-128, 128, (n, k), generator=g, dtype=torch.int8)
    return a, b


SHAPES = [
    (128, 256, 128),    # one tile, one K block
    (128, 128, 512),    # narrow-N kernel variant
    (256, 512, 640),    # K = 5 blocks (the SDXL FF K)
    (130, 72, 144),     # ragged in M, N and K (K % 128 != 0, N % 8 == 0)
    (1, 8, 16),         # smallest legal problem
    (300, 1000, 3072),  # deep K: phases wrap many times
    (4608, 640, 2560),  # many tiles per CTA on the narrow variant (SDXL FF-out shape)
    (515, 2050, 96),    # N % 8 != 0 -> scalar store path
]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_int32_accumulators_bit_exact(ops, tile, m, n, k):
    a, b = _rand_int8(m, n, k, seed=m + n + k)
    c = torch.full((m, n), -7, dtype=torch.int32, device="cuda")
    ops.run_gemm_int8(cu(a), cu(b), None, None, c)
    check_status()
    assert_bit_equal(c, gemm.int8_gemm_acc(a, b), "s32 accumulators %s" % ((m, n, k),))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (130, 72, 144), (700, 1280, 640)])
def test_dequant_epilogue_bit_exact(ops, tile, dtype, m, n, k):
    a, b = _rand_int8(m, n, k, seed=3 * m + n)
    g = torch.Generator().manual_seed(m)
    alpha_col = (torch.rand(n, generator=g) * 1e-3 + 1e-4).float()
    alpha_tok = (torch.rand(m, generator=g) * 1e-2 + 1e-3).float()
    alpha_one = torch.tensor([0.0071], dtype=torch.float32)
    bias = (torch.randn(n, generator=g) * 0.05).to(dtype)
    acc = gemm.int8_gemm_acc(a, b)
    c = torch.empty(m, n, dtype=dtype, device="cuda")
    for per_token, ar in ((False, alpha_one), (True, alpha_tok)):
        for bi in (None, bias):
            ops.run_gemm_int8(cu(a), cu(b), cu(alpha_col), cu(ar), c, bias=cu(bi), per_token=per_token)
            want = gemm.int8_gemm(a, b, alpha_col, ar, dtype, per_token=per_token, bias=bi, acc=acc)
            assert_bit_equal(c, want, "per_token=%s bias=%s" % (per_token, bi is not None))
    check_status()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (130, 72, 144), (520, 640, 2560)])
def test_residual_epilogue_bit_exact(ops, tile, dtype, m, n, k):
    """T(T(T(acc * scale) + R) + bias): the feed-forward output linear of the SDXL block with its residual add fused;
    also in place (C aliases R), which is how the reference's block calls it."""
    a, b = _rand_int8(m, n, k, seed=5 * m + n)
    g = torch.Generator().manual_seed(n)
    alpha_col = (torch.rand(n, generator=g) * 1e-3 + 1e-4).float()
    alpha_one = torch.tensor([0.0045], dtype=torch.float32)
    bias = (torch.randn(n, generator=g) * 0.05).to(dtype)
    res = torch.randn(m, n, generator=g).to(dtype)
    acc = gemm.int8_gemm_acc(a, b)
    c = torch.empty(m, n, dtype=dtype, device="cuda")
    for bi in (None, bias):
        ops.run_gemm_int8(cu(a), cu(b), cu(alpha_col), cu(alpha_one), c, bias=cu(bi), residual=cu(res))
        want = gemm.int8_gemm(a, b, alpha_col, alpha_one, dtype, bias=bi, acc=acc, residual=res)
        assert_bit_equal(c, want, "bias=%s" % (bi is not None))
    inplace = cu(res).clone()
    ops.run_gemm_int8(cu(a), cu(b), cu(alpha_col), cu(alpha_one), inplace, bias=cu(bias), residual=inplace)
    assert_bit_equal(inplace, gemm.int8_gemm(a, b, alpha_col, alpha_one, dtype, bias=bias, acc=acc, residual=res), "in place")
    check_status()


def test_golden_vectors(ops, golden):
    z = golden("int8")
    m, k = z["qa"].shape
    n = z["qw"].shape[0]
    c32 = torch.empty(m, n, dtype=torch.int32, device="cuda")
    ops.run_gemm_int8(cu(z["qa"]), cu(z["qw"]), None, None, c32)
    assert_bit_equal(c32, z["acc"])
    y = torch.empty(m, n, dtype=torch.float16, device="cuda")
    ops.run_gemm_int8(cu(z["qa"]), cu(z["qw"]), cu(z["s_w"]), cu(z["sa"]), y, bias=cu(z["bias"]), per_token=True)
    assert_bit_equal(y, z["y"])


def test_smoothquant_linear_end_to_end_small(ops):
    """quantize (dynamic per-token) -> GEMM -> dequant + bias, all on the device, equals the oracle chain."""
    wl = workloads.int8_smoothquant_linear(m=512, k=640, n=768, seed=1)
    x, pre = cu(wl["x"]), cu(wl["pre"])
    qa = torch.empty(512, 640, dtype=torch.int8, device="cuda")
    sa = torch.empty(512, dtype=torch.float32, device="cuda")
    ops.invoke_sq_input_quant(qa, x, pre, sa, dynamic=True)
    qw = torch.empty(768, 640, dtype=torch.int8, device="cuda")
    sw = torch.empty(768, dtype=torch.float32, device="cuda")
    ops.invoke_get_int8_weight_scale(sw, qw, cu(wl["w"]), pre)
    y = torch.empty(512, 768, dtype=torch.float16, device="cuda")
    ops.run_gemm_int8(qa, qw, sw, sa, y, bias=cu(wl["bias"]), per_token=True)
    q_ref, s_ref = quant.sq_input_quant_dynamic(wl["x"], wl["pre"])
    want = gemm.int8_gemm(q_ref, wl["qw"], wl["s_w"], s_ref, torch.float16, per_token=True, bias=wl["bias"])
    assert_bit_equal(y, want)
    ref = wl["x"].float() @ wl["w"].float().t() + wl["bias"].float()
    assert float((y.cpu().float() - ref).norm() / ref.norm()) < 0.03


def test_full_size_config1(ops):
    """The SDXL GEGLU feed-forward linear at full size (M=8192, K=640, N=5120): accumulators checked bit-exactly on a strided sample
    of rows and columns against the oracle, plus two size-independent properties: linearity in A
    (acc(A) + acc(-A) == 0) and a column checksum (sum_n acc[m,n] == A[m,:] . sum_n B[n,:])."""
    wl = workloads.int8_smoothquant_linear(seed=0)
    qa_ref, sa_ref = quant.sq_input_quant_dynamic(wl["x"], wl["pre"])
    qa = torch.empty(8192, 640, dtype=torch.int8, device="cuda")
    sa = torch.empty(8192, dtype=torch.float32, device="cuda")
    ops.invoke_sq_input_quant(qa, cu(wl["x"]), cu(wl["pre"]), sa, dynamic=True)
    assert_bit_equal(qa, qa_ref)
    assert_bit_equal(sa, sa_ref)
    qw = cu(wl["qw"])
    c = torch.empty(8192, 5120, dtype=torch.int32, device="cuda")
    ops.run_gemm_int8(qa, qw, None, None, c)
    rows = torch.arange(0, 8192, 61)
    assert_bit_equal(c[rows.cuda()], gemm.int8_gemm_acc(qa_ref[rows], wl["qw"]), "sampled rows")
    checksum = qa_ref.to(torch.int64) @ wl["qw"].to(torch.int64).sum(dim=0)
    assert torch.equal(c.sum(dim=1, dtype=torch.int64).cpu(), checksum)
    neg = torch.empty_like(c)
    ops.run_gemm_int8((-qa.to(torch.int16)).clamp(-128, 127).to(torch.int8), qw, None, None, neg)
    clean = (qa_ref != -128).all(dim=1).cuda()  # -(-128) saturates; leave those rows out
    assert int((c[clean] + neg[clean]).abs().max()) == 0
    y = torch.empty(8192, 5120, dtype=torch.float16, device="cuda")
    ops.run_gemm_int8(qa, qw, cu(wl["s_w"]), sa, y, bias=cu(wl["bias"]), per_token=True)
    want = gemm.int8_gemm(qa_ref[rows], wl["qw"], wl["s_w"], sa_ref[rows], torch.float16, per_token=True, bias=wl["bias"])
    assert_bit_equal(y[rows.cuda()], want, "fp16 output, sampled rows")
    check_status()
