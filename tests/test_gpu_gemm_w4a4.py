"""GPU parity tests of the W4A4 group-64 GEMM against the CPU oracle, through the C ABI.
With unit scales the fp32 output is the exact integer sum of the per-group int32 partials (bit-exact check of
the integer path, nibble expansion included).  With real scales the kernel follows the oracle's arithmetic
(t = float(p)*sa; acc = fma(t, sb, acc), groups in order), so fp32 and bf16 outputs are compared bit for bit."""

import pytest
import torch

from oracle import gemm, quant, workloads
from tests.util import assert_bit_equal, check_status, cu, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from lyradiff_b200 import ops as _ops
    return _ops


def _rand_int4(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    qa = torch.randint(-8, 8, (m, k), generator=g, dtype=torch.int8)
    qw = torch.randint(-8, 8, (n, k), generator=g, dtype=torch.int8)
    return qa, qw


SHAPES = [(128, 128, 128), (128, 128, 64), (130, 72, 192), (1, 8, 64), (260, 520, 3072), (384, 256, 12288)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_unit_scales_give_exact_integer_sums(ops, m, n, k):
    qa, qw = _rand_int4(m, n, k, seed=m * 3 + n + k)
    g = k // 64
    d = torch.full((m, n), -1.0, dtype=torch.float32, device="cuda")
    ops.invoke_fused_w4a4_gemm_and_lora_up(d, cu(quant.pack_int4(qa)), cu(quant.pack_int4(qw)), None, None,
                                           cu(torch.ones(m, g)), cu(torch.ones(n, g)))
    check_status()
    want = (qa.to(torch.int64) @ qw.to(torch.int64).t()).float()
    assert_bit_equal(d, want, "integer sums %s" % ((m, n, k),))


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (130, 72, 192), (260, 520, 3072)])
@pytest.mark.parametrize("sb_dtype", [torch.float32, torch.float16])
def test_group_rescale_bit_exact(ops, m, n, k, sb_dtype):
    qa, qw = _rand_int4(m, n, k, seed=m + n * 5 + k)
    g = torch.Generator().manual_seed(k)
    sa = (torch.rand(m, k // 64, generator=g) * 0.5 + 0.1).float()
    sb = (torch.rand(n, k // 64, generator=g) * 0.01 + 0.001).to(sb_dtype)
    pa, pw = cu(quant.pack_int4(qa)), cu(quant.pack_int4(qw))
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        d = torch.empty(m, n, dtype=dt, device="cuda")
        ops.invoke_fused_w4a4_gemm_and_lora_up(d, pa, pw, None, None, cu(sa), cu(sb))
        assert_bit_equal(d, gemm.w4a4_gemm(qa, qw, sa, sb, out_dtype=dt), str(dt))
    check_status()


def test_epilogues(ops):
    qa, qw = _rand_int4(200, 264, 256, seed=8)
    g = torch.Generator().manual_seed(8)
    sa = (torch.rand(200, 4, generator=g) * 0.5 + 0.1).float()
    sb = (torch.rand(264, 4, generator=g) * 0.01 + 0.001).float()
    bias = (torch.randn(264, generator=g) * 0.1).bfloat16()
    res = torch.randn(200, 264, generator=g).bfloat16()
    pa, pw = cu(quant.pack_int4(qa)), cu(quant.pack_int4(qw))
    d = torch.empty(200, 264, dtype=torch.bfloat16, device="cuda")
    ops.invoke_fused_w4a4_gemm_and_lora_up(d, pa, pw, None, None, cu(sa), cu(sb), bias=cu(bias), residual=cu(res))
    assert_bit_equal(d, gemm.w4a4_gemm(qa, qw, sa, sb, bias=bias, residual=res), "bias + residual")
    ops.invoke_fused_w4a4_gemm_and_lora_up(d, pa, pw, None, None, cu(sa), cu(sb), bias=cu(bias), is_gelu=True)
    want = gemm.w4a4_gemm(qa, qw, sa, sb, bias=bias, gelu=True)
    assert rel_err(d, want) < 5e-3  # tanh.approx.f32 on the device


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_round_each_step_matches_separate_kernels(ops, dt):
    """LYRAQ_EPI_ROUND_EACH: T after the accumulate, after the bias, (after GELU,) after the residual, i.e. the bits of the
    reference's GEMM followed by its separate 16-bit bias / residual kernels."""
    qa, qw = _rand_int4(200, 264, 256, seed=18)
    g = torch.Generator().manual_seed(18)
    sa = (torch.rand(200, 4, generator=g) * 0.5 + 0.1).float()
    sb = (torch.rand(264, 4, generator=g) * 0.01 + 0.001).float()
    bias = (torch.randn(264, generator=g) * 0.1).to(dt)
    res = torch.randn(200, 264, generator=g).to(dt)
    pa, pw = cu(quant.pack_int4(qa)), cu(quant.pack_int4(qw))
    d = torch.empty(200, 264, dtype=dt, device="cuda")
    ops.invoke_fused_w4a4_gemm_and_lora_up(d, pa, pw, None, None, cu(sa), cu(sb), bias=cu(bias), residual=cu(res), round_each=True)
    want = gemm.w4a4_gemm(qa, qw, sa, sb, out_dtype=dt, bias=bias, residual=res, round_each=True)
    assert_bit_equal(d, want, "round each: bias + residual")
    once = gemm.w4a4_gemm(qa, qw, sa, sb, out_dtype=dt, bias=bias, residual=res)
    assert not torch.equal(want, once)  # the two roundings do differ on this input
    ops.invoke_fused_w4a4_gemm_and_lora_up(d, pa, pw, None, None, cu(sa), cu(sb), bias=cu(bias), is_gelu=True, round_each=True)
    want = gemm.w4a4_gemm(qa, qw, sa, sb, out_dtype=dt, bias=bias, gelu=True, round_each=True)
    assert rel_err(d, want) < 5e-3  # tanh.approx.f32 on the device
    check_status()


def test_golden_vectors(ops, golden):
    z = golden("w4a4")
    m, n = z["packed_a"].shape[0], z["packed_w"].shape[0]
    d = torch.empty(m, n, dtype=torch.float32, device="cuda")
    ops.invoke_fused_w4a4_gemm_and_lora_up(d, cu(z["packed_a"]), cu(z["packed_w"]), None, None, cu(z["sa"]), cu(z["s_w"]))
    assert_bit_equal(d, z["y_f32"])
    db = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ops.invoke_fused_w4a4_gemm_and_lora_up(db, cu(z["packed_a"]), cu(z["packed_w"]), None, None, cu(z["sa"]), cu(z["s_w"]))
    assert_bit_equal(db, z["y_bf16"])


def test_quantize_then_gemm_end_to_end(ops):
    w = workloads.w4a4_linear(m=256, k=3072, n=384, seed=5, smooth_nontrivial=True)
    x = cu(w["x"])
    q = torch.empty(256, 1536, dtype=torch.uint8, device="cuda")
    s = torch.empty(256, 48, dtype=torch.float32, device="cuda")
    ops.invoke_fused_quantize_and_lora_down_simple(None, q, s, x, None, cu(w["smooth"]))
    qw = torch.empty(384, 1536, dtype=torch.uint8, device="cuda")
    sw = torch.empty(384, 48, dtype=torch.float16, device="cuda")
    ops.weight_quant_int4_g64(qw, sw, cu(w["w"]))
    d = torch.empty(256, 384, dtype=torch.bfloat16, device="cuda")
    ops.invoke_fused_w4a4_gemm_and_lora_up(d, q, qw, None, None, s, sw)
    pa, sa, qa = quant.int4_quant_g64(w["x"], w["smooth"])
    assert_bit_equal(d, gemm.w4a4_gemm(qa, w["qw"], sa, w["s_w"]))
    ref = (w["x"].float() / w["smooth"]) @ w["w"].float().t()
    assert rel_err(d, ref) < 0.25  # int4 x int4 quantization noise


def test_full_size_config3(ops):
    """The fused FLUX W4A4 projection at full size (M=4608, K=3072, N=21504): sampled rows bit-exact against the oracle, and the
    exact-integer property with unit scales on the full problem via a column checksum."""
    w = workloads.w4a4_linear(seed=0)
    pa, sa, qa = quant.int4_quant_g64(w["x"], w["smooth"])
    A, B = cu(pa), cu(w["packed_w"])
    d = torch.empty(4608, 21504, dtype=torch.bfloat16, device="cuda")
    ops.invoke_fused_w4a4_gemm_and_lora_up(d, A, B, None, None, cu(sa), cu(w["s_w"]))
    rows = torch.arange(0, 4608, 307)
    assert_bit_equal(d[rows.cuda()], gemm.w4a4_gemm(qa[rows], w["qw"], sa[rows], w["s_w"]), "sampled rows")
    d32 = torch.empty(4608, 21504, dtype=torch.float32, device="cuda")
    ops.invoke_fused_w4a4_gemm_and_lora_up(d32, A, B, None, None, cu(torch.ones(4608, 48)), cu(torch.ones(21504, 48)))
    checksum = qa.to(torch.int64) @ w["qw"].to(torch.int64).sum(dim=0)
    assert torch.equal(d32.sum(dim=1, dtype=torch.float64).to(torch.int64).cpu(), checksum)
    check_status()


@pytest.mark.parametrize("m,k", [(32, 64), (100, 192), (260, 3072), (4608, 3072)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_lora_down_next_to_the_quantize(ops, m, k, dt):
    """act = x * lora_down^T in fp32 (tensor-core accumulation order is the hardware's: tolerance 2e-5 of the row's
    absolute sum); q and scales are the same as without the low-rank branch."""
    g = torch.Generator().manual_seed(m + k)
    x = torch.randn(m, k, generator=g).to(dt)
    down = (torch.randn(32, k, generator=g) * 0.05).to(dt)
    smooth = (torch.rand(k, generator=g) + 0.5).float()
    q = torch.empty(m, k // 2, dtype=torch.uint8, device="cuda")
    s = torch.empty(m, k // 64, dtype=torch.float32, device="cuda")
    act = torch.full((m, 32), float("nan"), dtype=torch.float32, device="cuda")
    ops.invoke_fused_quantize_and_lora_down_simple(act, q, s, cu(x), cu(down), cu(smooth))
    check_status()
    want_q, want_s, _ = quant.int4_quant_g64(x, smooth)
    assert_bit_equal(q, want_q, "packed int4")
    assert_bit_equal(s, want_s, "group scales")
    want = quant.lora_down(x, down)
    bound = 2e-5 * (x.double().abs() @ down.double().abs().t()).float() + 1e-30
    err = (act.cpu() - want).abs()
    assert bool((err <= bound).all()), "lora_down: worst error / bound = %g" % float((err / bound).max())
    # reproducible: a second run gives the same bits
    act2 = torch.empty_like(act)
    ops.invoke_fused_quantize_and_lora_down_simple(act2, q, s, cu(x), cu(down), cu(smooth))
    assert_bit_equal(act2, act.cpu(), "second run")


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (130, 72, 192), (260, 520, 3072)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_lora_up_added_after_the_groups(ops, m, n, k, dt):
    """D = T(groups + T(act) * up^T): the low-rank term is a 32-term fp32 tensor-core sum added to the accumulator once,
    so the result may differ from the oracle's single rounding by an fp32 ulp before the rounding to T: at most one
    T ulp (plus the fp32 rounding of terms that cancel) on at most 1 % of the outputs."""
    qa, qw = _rand_int4(m, n, k, seed=m + n + k + 1)
    g = torch.Generator().manual_seed(n)
    sa = (torch.rand(m, k // 64, generator=g) * 0.5 + 0.1).float()
    sb = (torch.rand(n, k // 64, generator=g) * 0.01 + 0.001).float()
    act = torch.randn(m, 32, generator=g).float() * 3.0
    up = (torch.randn(n, 32, generator=g) * 0.3).to(dt)
    bias = (torch.randn(n, generator=g) * 0.1).to(dt)
    d = torch.empty(m, n, dtype=dt, device="cuda")
    ops.invoke_fused_w4a4_gemm_and_lora_up(d, cu(quant.pack_int4(qa)), cu(quant.pack_int4(qw)), cu(act), cu(up), cu(sa), cu(sb),
                                           bias=cu(bias))
    check_status()
    want = gemm.w4a4_gemm(qa, qw, sa, sb, out_dtype=dt, lora_act=act, lora_up=up, bias=bias)
    base = gemm.w4a4_gemm(qa, qw, sa, sb, out_dtype=dt, bias=bias)
    assert not torch.equal(want, base)  # the low-rank term matters in this test
    got = d.cpu()
    diff = (got.float() - want.float()).abs()
    # one ulp of T at the result, plus the fp32 rounding of the larger terms the result was summed from (they may cancel)
    terms = (gemm.w4a4_gemm(qa, qw, sa, sb, out_dtype=torch.float32).abs() + bias.float().abs()[None, :] +
             (act.to(dt).float() @ up.float().t()).abs())
    bound = torch.finfo(dt).eps * want.float().abs() + 2.0 ** -22 * terms
    assert bool((diff <= bound).all()), "worst = %g of the bound" % float((diff / bound).max())
    assert float((diff > 0).float().mean()) <= 1e-2
    # the reference's caller converts act to T first and passes that: same bits
    d2 = torch.empty_like(d)
    ops.invoke_fused_w4a4_gemm_and_lora_up(d2, cu(quant.pack_int4(qa)), cu(quant.pack_int4(qw)), cu(act.to(dt)), cu(up), cu(sa),
                                           cu(sb), bias=cu(bias))
    assert_bit_equal(d2, got, "act already of type T")


def test_lora_pointers_must_come_together(ops):
    from lyradiff_b200 import _lib
    d = torch.empty(128, 128, dtype=torch.bfloat16, device="cuda")
    a = torch.zeros(128, 32, dtype=torch.uint8, device="cuda")
    s = torch.ones(128, 1, dtype=torch.float32, device="cuda")
    act = torch.zeros(128, 32, dtype=torch.float32, device="cuda")
    with pytest.raises(_lib.LyraqError):
        ops.invoke_fused_w4a4_gemm_and_lora_up(d, a, a, act, None, s, s)
    d32 = torch.empty(128, 128, dtype=torch.float32, device="cuda")
    up = torch.zeros(128, 32, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.LyraqError):
        ops.invoke_fused_w4a4_gemm_and_lora_up(d32, a, a, act, up, s, s)  # fp32 output has no 16-bit type for lora_up
