"""GPU parity tests of lyraq_attention (tcgen05 attention forward over the packed QKV projection) against the CPU
oracle's exact attention (oracle/blocks.py::attention, fp64 softmax), through the C ABI."""

import pytest
import torch

from oracle import blocks, quant
from tests.util import assert_bit_equal, check_status, cu

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from lyradiff_b200 import ops as _ops
    return _ops


def _oracle(qkv, batch, seq, heads, head_dim):
    x = qkv.reshape(batch, seq, 3, heads, head_dim).permute(2, 0, 3, 1, 4)          # [3, B, H, S, Dh]
    o = blocks.attention(x[0], x[1], x[2])                                          # [B, H, S, Dh] fp64
    return o.permute(0, 2, 1, 3).reshape(batch * seq, heads * head_dim)


def _qkv(batch, seq, heads, head_dim, dtype, g, spread=1.0):
    """q and k with unit RMS per head (what QK RMSNorm leaves), v ~ N(0, 1); `spread` widens the score range."""
    x = torch.randn(batch * seq, 3, heads, head_dim, generator=g)
    x[:, 0] *= spread
    return x.reshape(batch * seq, 3 * heads * head_dim).to(dtype)


# Tolerance.  Scores and sums are fp32; the probabilities are rounded to the 16-bit type before the second product
# (half an ulp each, signs random, so their effect on a row is about one rounding of the output) and the result is
# rounded to that type once more.  With eps = one ulp of T at 1: stated bound max |err| <= 2.5 eps max|want| and
# mean |err| <= 0.5 eps mean|want| (a single correct rounding alone gives about 0.2 eps mean|want|).
def _check(got, want, dtype):
    eps = torch.finfo(dtype).eps
    err = (got.double() - want).abs()
    assert float(err.max()) <= 2.5 * eps * float(want.abs().max()), (float(err.max()), float(want.abs().max()))
    assert float(err.mean()) <= 0.5 * eps * float(want.abs().mean()), (float(err.mean()), float(want.abs().mean()))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("batch,seq,heads", [(1, 256, 2), (1, 128, 1), (1, 100, 2), (2, 300, 3), (1, 777, 2), (3, 64, 1)])
def test_attention_against_oracle(ops, dtype, batch, seq, heads):
    g = torch.Generator().manual_seed(seq * 7 + heads)
    qkv = _qkv(batch, seq, heads, 128, dtype, g)
    want = _oracle(qkv, batch, seq, heads, 128)
    out = torch.full((batch * seq, heads * 128), float("nan"), dtype=dtype, device="cuda")
    ops.flash_attention(cu(qkv), batch, seq, heads, 128, out=out)
    check_status()
    got = out.cpu()
    assert bool(torch.isfinite(got.float()).all())
    _check(got, want, dtype)


def test_attention_wide_scores_and_rescale(ops):
    """Scores spread over tens of units: the running maximum moves by more than the lazy-rescale threshold between
    key tiles, so the accumulator rescale in tensor memory runs; large positive and negative scores, nothing overflows."""
    g = torch.Generator().manual_seed(5)
    batch, seq, heads = 1, 1024, 2
    qkv = _qkv(batch, seq, heads, 128, torch.bfloat16, g, spread=6.0)
    # rows whose best key comes late: make the keys of the last tile align with the queries
    x = qkv.reshape(seq, 3, heads, 128).clone()
    x[:, 1][900:] = (x[:, 0][:124] * 0.5).to(x.dtype)
    qkv = x.reshape(seq, 3 * heads * 128)
    want = _oracle(qkv, batch, seq, heads, 128)
    out = torch.empty(seq, heads * 128, dtype=torch.bfloat16, device="cuda")
    ops.flash_attention(cu(qkv), batch, seq, heads, 128, out=out)
    check_status()
    _check(out.cpu(), want, torch.bfloat16)


def test_attention_e4m3_output_into_a_column_window_and_split(ops):
    """The fused quantize equals quantizing the 16-bit result (same rounding to T first, then 1 / scale and e4m3), the
    window leaves the other columns alone, and rows from `split` on land in the second output with its own scale."""
    g = torch.Generator().manual_seed(9)
    batch, seq, heads, split = 2, 200, 2, 72
    width = heads * 128
    qkv = cu(_qkv(batch, seq, heads, 128, torch.bfloat16, g))
    ref16 = torch.empty(batch * seq, width, dtype=torch.bfloat16, device="cuda")
    ops.flash_attention(qkv, batch, seq, heads, 128, out=ref16)
    s1 = torch.tensor([0.02], device="cuda")
    s2 = torch.tensor([0.013], device="cuda")
    # one output, window at column 128 of a wider matrix
    wide = torch.full((batch * seq, width + 384), 0x55, dtype=torch.uint8, device="cuda")
    ops.flash_attention(qkv, batch, seq, heads, 128, out=wide, out_scale=s1, col0=128)
    check_status()
    want = quant.fp8_quant(ref16.cpu(), s1.cpu())
    assert_bit_equal(wide[:, 128:128 + width], want, "e4m3 window")
    assert int((wide[:, :128] != 0x55).sum()) == 0 and int((wide[:, 128 + width:] != 0x55).sum()) == 0
    # two outputs
    a = torch.zeros(batch * split, width, dtype=torch.uint8, device="cuda")
    b = torch.zeros(batch * (seq - split), width + 128, dtype=torch.uint8, device="cuda")
    ops.flash_attention(qkv, batch, seq, heads, 128, out=a, out_scale=s1, out2=b, out2_scale=s2, col0_2=128, split=split)
    check_status()
    r = ref16.cpu().reshape(batch, seq, width)
    assert_bit_equal(a, quant.fp8_quant(r[:, :split].reshape(-1, width), s1.cpu()), "text part")
    assert_bit_equal(b[:, 128:], quant.fp8_quant(r[:, split:].reshape(-1, width), s2.cpu()), "image part")
    # 16-bit split
    a16 = torch.empty(batch * split, width, dtype=torch.bfloat16, device="cuda")
    b16 = torch.empty(batch * (seq - split), width, dtype=torch.bfloat16, device="cuda")
    ops.flash_attention(qkv, batch, seq, heads, 128, out=a16, out2=b16, split=split)
    assert_bit_equal(a16, r[:, :split].reshape(-1, width), "text part 16-bit")
    assert_bit_equal(b16, r[:, split:].reshape(-1, width), "image part 16-bit")


def test_attention_flux_size_sample_and_properties(ops):
    """4608 tokens, 24 heads (the FLUX.1-dev shape): a strided sample of query rows against the oracle (which needs all
    keys but only the sampled queries), run-to-run identical bits, and the convexity property: every output lies inside
    the range of its head's v columns."""
    g = torch.Generator().manual_seed(21)
    seq, heads = 4608, 24
    qkv = _qkv(1, seq, heads, 128, torch.bfloat16, g)
    dq = cu(qkv)
    out = torch.empty(seq, heads * 128, dtype=torch.bfloat16, device="cuda")
    ops.flash_attention(dq, 1, seq, heads, 128, out=out)
    check_status()
    out2 = torch.empty_like(out)
    ops.flash_attention(dq, 1, seq, heads, 128, out=out2)
    assert_bit_equal(out2, out.cpu(), "run to run")
    x = qkv.reshape(seq, 3, heads, 128)
    rows = torch.arange(0, seq, 97)
    for h in (0, 11, 23):
        q, k, v = x[rows, 0, h].double(), x[:, 1, h].double(), x[:, 2, h].double()
        want = torch.softmax(q @ k.t() / 128 ** 0.5, dim=-1) @ v
        got = out.cpu()[rows, h * 128:(h + 1) * 128]
        _check(got, want, torch.bfloat16)
        vmax, vmin = x[:, 2, h].float().max(dim=0).values, x[:, 2, h].float().min(dim=0).values
        o = out.cpu()[:, h * 128:(h + 1) * 128].float()
        assert bool((o <= vmax + 1e-2).all()) and bool((o >= vmin - 1e-2).all())


def test_attention_argument_checks():
    from lyradiff_b200 import _lib
    lib = _lib.lib()
    p = 1 << 20
    assert lib.lyraq_attention(None, 1, 256, None, None, 0, None, 0, None, 1, 1, 8, 2, 128, 0.1, None) == 1
    assert lib.lyraq_attention(p, 1, 256, None, None, 0, None, 0, p, 1, 1, 8, 2, 64, 0.1, None) == 2       # head_dim 128 only
    assert lib.lyraq_attention(p, 1, 256, None, None, 0, None, 0, p, 2, 1, 8, 2, 128, 0.1, None) == 2      # fp32
    assert lib.lyraq_attention(p, 4, 256, None, None, 0, None, 0, p, 1, 1, 8, 2, 128, 0.1, None) == 1      # e4m3 without a scale
    assert lib.lyraq_attention(p, 1, 128, None, None, 0, None, 0, p, 1, 1, 8, 2, 128, 0.1, None) == 1      # pitch below the width
    assert lib.lyraq_attention(p, 1, 256, None, None, 0, None, 0, p, 1, 0, 8, 2, 128, 0.1, None) == 0      # empty


def test_a_wait_that_runs_out_is_reported_and_the_kernel_returns(ops):
    """Nothing faults or hangs here: a test hook makes the producer issue no copy and shortens the wait limit to 50 ms, so
    the consumers' waits run out.  The kernel must come back, leave LYRAQ_ERR_DEVICE_TIMEOUT (4) with the code of an
    attention wait (0x3xxx) in the status word, write nothing -- and the next ordinary call must work and give the usual
    bits (the abort path freed tensor memory and left no copy in flight)."""
    from lyradiff_b200 import _lib
    lib = _lib.lib()
    g = torch.Generator().manual_seed(3)
    qkv = cu(_qkv(1, 256, 2, 128, torch.bfloat16, g))
    good = torch.empty(256, 256, dtype=torch.bfloat16, device="cuda")
    ops.flash_attention(qkv, 1, 256, 2, 128, out=good)
    check_status()
    out = torch.full((256, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    assert lib.lyraq_debug_attention_wait_test(1, 50) == 0
    try:
        ops.flash_attention(qkv, 1, 256, 2, 128, out=out)          # the launch itself succeeds
        torch.cuda.synchronize()
        status, detail = ops.last_status()
    finally:
        assert lib.lyraq_debug_attention_wait_test(0, 0) == 0
    assert status == 4, status
    assert 0x3000 <= detail < 0x4000, hex(detail)
    assert bool((out == 7.0).all()), "a timed-out kernel must not store results"
    assert ops.last_status()[0] == 0                               # reading the status cleared it
    again = torch.empty_like(good)
    ops.flash_attention(qkv, 1, 256, 2, 128, out=again)
    check_status()
    assert_bit_equal(again, good.cpu(), "after a timed-out launch")
