"""GPU parity tests of the FP8 e4m3 tcgen05 GEMM against the CPU oracle (fp64 contraction), through the C ABI.
Stated tolerance: relative Frobenius error <= 1e-2 of the bf16/fp16 output (the reference arithmetic is a closed
library; the measured error is in fact near bf16 rounding, ~2e-3), and element-wise |d| <= 2 output ulps + 1e-2*|y|."""

import pytest
import torch

from oracle import gemm, quant, workloads
from tests.util import check_status, cu, rel_err

pytestmark = pytest.mark.gpu

REL_TOL = 1e-2


@pytest.fixture(scope="module")
def ops():
    from lyradiff_b200 import ops as _ops
    return _ops


@pytest.fixture(params=[0, 2561, 1281, 2562], ids=["auto", "1cta_n256", "1cta_n128", "pair_n256"])
def tile(request):
    from lyradiff_b200 import _lib
    assert _lib.lib().lyraq_debug_force_gemm_tile(request.param) == 0
    yield request.param
    _lib.lib().lyraq_debug_force_gemm_tile(0)


def _run(ops, f, dtype, bias=True, residual=False, gelu=False, alpha=1.0, beta=1.0):
    m, k = f["qx"].shape
    n = f["qw"].shape[0]
    y = torch.empty(m, n, dtype=dtype, device="cuda")
    b = f["bias"].to(dtype) if bias else None
    r = f["residual"].to(dtype) if residual else None
    ops.gemm_with_residual_and_bias_fp8(cu(f["qw"]), cu(f["s_w"]), cu(f["qx"]), cu(f["s_x"]), y, bias=cu(b), residual=cu(r),
                                        alpha=alpha, beta=beta, is_gelu=gelu)
    want = gemm.fp8_gemm(f["qx"], f["qw"], f["s_x"], f["s_w"], out_dtype=dtype, bias=b, residual=r, alpha=alpha, beta=beta,
                         gelu=gelu)
    return y, want


def _check(y, want, dtype):
    assert rel_err(y, want) <= REL_TOL
    ulp = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -20}[dtype]
    d = (y.cpu().double() - want.double()).abs()
    bound = 2 * ulp * want.double().abs() + 1e-2 * want.double().abs() + 1e-3
    assert bool((d <= bound).all()), float((d - bound).max())


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (128, 128, 256), (130, 72, 144), (1, 8, 16), (300, 1000, 3072),
                                   (256, 384, 12288)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_plain_and_bias(ops, tile, m, n, k, dtype):
    f = workloads.fp8_linear(m, k, n, seed=m + n, with_residual=True)
    for bias in (False, True):
        y, want = _run(ops, f, dtype, bias=bias)
        _check(y, want, dtype)
    check_status()


def test_exact_on_small_integers(ops, tile):
    """Operands that are small integers in e4m3 and unit scales give integer sums below 2**24: fp32 accumulation
    must then be exact, whatever the order."""
    g = torch.Generator().manual_seed(4)
    xi = torch.randint(-8, 9, (200, 512), generator=g).float()
    wi = torch.randint(-8, 9, (136, 512), generator=g).float()
    one = torch.ones(1)
    qx, qw = quant.fp8_quant(xi, one), quant.fp8_quant(wi, one)
    y = torch.empty(200, 136, dtype=torch.float32, device="cuda")
    ops.gemm_with_residual_and_bias_fp8(cu(qw), cu(one), cu(qx), cu(one), y)
    assert torch.equal(y.cpu(), xi @ wi.t())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gelu_and_residual_epilogues(ops, tile, dtype):
    f = workloads.fp8_linear(260, 512, 392, seed=21, with_residual=True)
    for kw in ({"gelu": True}, {"gelu": True, "bias": False}, {"residual": True}, {"residual": True, "beta": 0.5, "alpha": 2.0}):
        y, want = _run(ops, f, dtype, **kw)
        _check(y, want, dtype)
    check_status()


def test_golden_vectors(ops, golden):
    z = golden("fp8")
    f = {k: z[k] for k in ("qx", "qw", "s_x", "s_w", "bias", "residual")}
    for key, kw in (("y_plain", {}), ("y_gelu", {"gelu": True}), ("y_residual", {"residual": True})):
        y, _ = _run(ops, f, torch.bfloat16, **kw)
        _check(y, z[key], torch.bfloat16)


def test_quantize_then_gemm_matches_unquantized_linear(ops):
    f = workloads.fp8_linear(512, 3072, 640, seed=2)
    x, w = cu(f["x"]), cu(f["w"])
    sx = torch.zeros(1, dtype=torch.float32, device="cuda")
    sw = torch.zeros(1, dtype=torch.float32, device="cuda")
    ops.invoke_get_fp8_weight_scale(sx, x)
    ops.invoke_get_fp8_weight_scale(sw, w)
    qx = torch.empty(512, 3072, dtype=torch.uint8, device="cuda")
    qw = torch.empty(640, 3072, dtype=torch.uint8, device="cuda")
    ops.invoke_cuda_d2d_scale_cpy_convert(qx, x, sx)
    ops.invoke_cuda_d2d_scale_cpy_convert(qw, w, sw)
    assert torch.equal(qx.cpu(), f["qx"]) and torch.equal(qw.cpu(), f["qw"])
    y = torch.empty(512, 640, dtype=torch.bfloat16, device="cuda")
    ops.gemm_with_residual_and_bias_fp8(qw, sw, qx, sx, y, bias=cu(f["bias"]))
    ref = f["x"].float() @ f["w"].float().t() + f["bias"].float()
    assert rel_err(y, ref) < 0.05  # e4m3 quantization noise of both operands


@pytest.mark.parametrize("name,k,n,gelu,residual", workloads.FLUX_FP8_LINEARS)
def test_full_size_flux_linears(ops, name, k, n, gelu, residual):
    """The FLUX FP8 linears at full size (M=4608): a strided sample of rows against the oracle, and the
    row-checksum property sum_n Y[m,n] == s * X[m,:] . sum_n W[n,:] (fp32 output, no epilogue)."""
    m = workloads.FLUX_TOKENS
    f = workloads.fp8_linear(m, k, n, seed=7, with_bias=True, with_residual=residual)
    qx, qw, sx, sw = cu(f["qx"]), cu(f["qw"]), cu(f["s_x"]), cu(f["s_w"])
    y = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ops.gemm_with_residual_and_bias_fp8(qw, sw, qx, sx, y, bias=cu(f["bias"]), residual=cu(f["residual"]), is_gelu=gelu)
    rows = torch.arange(0, m, 149)
    want = gemm.fp8_gemm(f["qx"][rows], f["qw"], f["s_x"], f["s_w"], bias=f["bias"],
                         residual=None if f["residual"] is None else f["residual"][rows], gelu=gelu)
    _check(y[rows.cuda()], want, torch.bfloat16)
    y32 = torch.empty(m, n, dtype=torch.float32, device="cuda")
    ops.gemm_with_residual_and_bias_fp8(qw, sw, qx, sx, y32)
    wsum = quant.fp8_dequant(f["qw"]).double().sum(dim=0)
    check = (quant.fp8_dequant(f["qx"]).double() @ wsum) * float(f["s_x"]) * float(f["s_w"])
    got = y32.double().sum(dim=1).cpu()
    scale = (quant.fp8_dequant(f["qx"]).double().abs() @ quant.fp8_dequant(f["qw"]).double().abs().sum(dim=0)) * float(f["s_x"]) * float(f["s_w"])
    assert float(((got - check).abs() / scale).max()) < 1e-5
    check_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", [(260, 520, 512), (128, 256, 3072), (130, 72, 144)])
def test_fused_output_quantize(ops, tile, dtype, m, n, k):
    """The GEMM epilogue that also quantizes its result for the next FP8 linear equals GEMM -> T -> e4m3 quantize.
    A one-ulp difference of the T value (fp32 vs fp64 accumulation) can move an e4m3 code by one step: stated tolerance
    |code distance| <= 1 on <= 2 % of the outputs, everything else identical."""
    f = workloads.fp8_linear(m, k, n, seed=m + 3 * n, with_residual=True)
    y_scale = torch.tensor([0.037], dtype=torch.float32)
    for kw in ({"gelu": True}, {"residual": True}, {}):
        b = f["bias"].to(dtype)
        r = f["residual"].to(dtype) if kw.get("residual") else None
        yq = torch.empty(m, n, dtype=torch.uint8, device="cuda")
        ops.gemm_fp8_quant_out(cu(f["qw"]), cu(f["s_w"]), cu(f["qx"]), cu(f["s_x"]), yq, cu(y_scale), dtype, bias=cu(b),
                               residual=cu(r), is_gelu=bool(kw.get("gelu")))
        y = gemm.fp8_gemm(f["qx"], f["qw"], f["s_x"], f["s_w"], out_dtype=dtype, bias=b, residual=r, gelu=bool(kw.get("gelu")))
        want = quant.fp8_quant(y, y_scale)
        got = yq.cpu()
        same_sign = ((got ^ want) & 0x80) == 0
        dist = ((got & 0x7F).to(torch.int32) - (want & 0x7F).to(torch.int32)).abs()
        zeroish = ((got & 0x7F) <= 1) & ((want & 0x7F) <= 1)   # +-0 and the smallest subnormal may swap sign
        assert bool(((dist <= 1) & (same_sign | zeroish)).all())
        assert float((got != want).float().mean()) <= 0.02
    check_status()
