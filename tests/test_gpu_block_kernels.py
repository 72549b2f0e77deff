"""GPU parity tests of the kernels between the quantized linears of a FLUX block (QK RMSNorm + RoPE, e4m3 quantize into
a column window, gate + residual, GEMM with a strided e4m3 output) against the CPU oracle, through the C ABI."""

import pytest
import torch

from oracle import gemm, norms, quant, workloads
from tests.util import assert_bit_equal, check_status, cu

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from lyradiff_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("batch,seq,heads,head_dim", [(1, 7, 2, 128), (2, 33, 24, 128), (1, 50, 3, 64)])
def test_rmsnorm_rope_against_oracle(ops, dtype, batch, seq, heads, head_dim):
    """Device statistics are fp32 shuffle sums and rsqrtf (2 ulp): a result may sit on the other side of a rounding
    boundary of T, so at most 0.5 % of the outputs may differ, by at most 2 ulp of T at the head's amplitude; V heads
    and the out-of-place / in-place forms are bit-identical."""
    g = torch.Generator().manual_seed(batch * 100 + seq + heads)
    tokens = batch * seq
    qkv = torch.randn(tokens, 3 * heads * head_dim, generator=g).to(dtype)
    scale = (1.0 + 0.2 * torch.randn(2 * head_dim, generator=g)).to(dtype)
    ang = torch.rand(tokens, head_dim // 2, generator=g) * 6.28
    rope = torch.stack([torch.cos(ang), -torch.sin(ang), torch.sin(ang), torch.cos(ang)], dim=-1).to(dtype)
    want = norms.rmsnorm_rope(qkv, scale, rope, heads, head_dim, eps=1e-6)
    out = torch.full_like(qkv, float("nan"), device="cuda")
    ops.invoke_fused_rmsnorm_and_rope(out, cu(qkv), cu(scale), cu(rope), 1e-6, batch, seq, heads, head_dim)
    check_status()
    got = out.cpu()
    hd = heads * head_dim
    assert_bit_equal(got[:, 2 * hd:], want[:, 2 * hd:], "v heads are copied")
    diff = (got[:, :2 * hd].float() - want[:, :2 * hd].float()).abs()
    assert float(diff.max()) <= 2 * torch.finfo(dtype).eps * 8.0
    assert float((diff > 0).float().mean()) <= 5e-3
    inplace = cu(qkv).clone()
    ops.invoke_fused_rmsnorm_and_rope(inplace, inplace, cu(scale), cu(rope), 1e-6, batch, seq, heads, head_dim)
    assert_bit_equal(inplace, got, "in place")


def test_rmsnorm_rope_with_the_reference_table_fixture(ops):
    """The rotary table of tests/golden/ref_rope_table.npz came out of the reference's own rope / EmbedND; fed to
    lyraq_rmsnorm_rope in that [S, 64, 2, 2] layout (cast to the model type as the reference's wrapper does) the kernel
    must agree with the oracle under the tolerance of the test above, and the library's own table builder must give
    the kernel the same bits."""
    import os
    import numpy as np
    from lyradiff_b200 import rope as rope_host
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_rope_table.npz"))
    table = torch.from_numpy(z["table"])[0, 0].bfloat16()
    S, heads, head_dim = table.shape[0], 4, 128
    g = torch.Generator().manual_seed(12)
    qkv = torch.randn(S, 3 * heads * head_dim, generator=g).bfloat16()
    scale = (1.0 + 0.2 * torch.randn(2 * head_dim, generator=g)).bfloat16()
    want = norms.rmsnorm_rope(qkv, scale, table, heads, head_dim, eps=1e-6)
    out = torch.empty_like(qkv, device="cuda")
    ops.invoke_fused_rmsnorm_and_rope(out, cu(qkv), cu(scale), cu(table), 1e-6, 1, S, heads, head_dim)
    check_status()
    diff = (out.cpu().float() - want.float()).abs()
    assert float(diff.max()) <= 2 * torch.finfo(torch.bfloat16).eps * 8.0
    assert float((diff > 0).float().mean()) <= 5e-3
    own = rope_host.flux_rope_table(torch.from_numpy(z["ids"]))[0, 0].bfloat16()
    out2 = torch.empty_like(qkv, device="cuda")
    ops.invoke_fused_rmsnorm_and_rope(out2, cu(qkv), cu(scale), cu(own), 1e-6, 1, S, heads, head_dim)
    assert_bit_equal(out2, out.cpu(), "library-built table")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gate_residual_bit_exact(ops, dtype):
    g = torch.Generator().manual_seed(3)
    y = torch.randn(2, 37, 3072, generator=g).to(dtype)
    x = torch.randn(2, 37, 3072, generator=g).to(dtype)
    gate = torch.randn(2, 3072, generator=g).to(dtype)
    out = torch.empty_like(y, device="cuda")
    ops.invoke_fused_gate_and_residual(out, cu(y), cu(gate), cu(x))
    check_status()
    assert_bit_equal(out, norms.gate_residual(y, gate, x))


def test_quantize_into_a_column_window(ops):
    g = torch.Generator().manual_seed(4)
    a = torch.randn(130, 256, generator=g).bfloat16()
    s = torch.tensor([0.031], dtype=torch.float32)
    dst = torch.full((130, 1024), 0x7F, dtype=torch.uint8, device="cuda")
    ops.quant_fp8_into_columns(dst, 512, cu(a), cu(s))
    check_status()
    got = dst.cpu()
    assert_bit_equal(got[:, 512:768], quant.fp8_quant(a, s, invert_scale=True))
    assert bool((got[:, :512] == 0x7F).all()) and bool((got[:, 768:] == 0x7F).all())


@pytest.mark.parametrize("m,n,k,ld,col0", [(128, 256, 128, 512, 256), (200, 1024, 384, 1280, 256), (130, 72, 144, 80, 0)])
def test_gemm_with_strided_e4m3_output(ops, m, n, k, ld, col0):
    """lyraq_gemm_fp8_quant_ld writes the same codes as the contiguous form, at the row pitch asked for, and nothing
    outside its window (the last shape has a pitch that is not a multiple of 16: the direct-store path)."""
    w = workloads.fp8_linear(m=m, k=k, n=n, seed=m + n)
    ys = torch.tensor([0.05], dtype=torch.float32)
    ref = torch.empty(m, n, dtype=torch.uint8, device="cuda")
    ops.gemm_fp8_quant_out(cu(w["qw"]), cu(w["s_w"]), cu(w["qx"]), cu(w["s_x"]), ref, cu(ys), torch.bfloat16, bias=cu(w["bias"]),
                           is_gelu=True)
    dst = torch.full((m, ld), 0x55, dtype=torch.uint8, device="cuda")
    ops.gemm_fp8_quant_into_columns(cu(w["qw"]), cu(w["s_w"]), cu(w["qx"]), cu(w["s_x"]), dst, col0, cu(ys), torch.bfloat16,
                                    bias=cu(w["bias"]), is_gelu=True)
    check_status()
    got = dst.cpu()
    assert_bit_equal(got[:, col0:col0 + n], ref.cpu())
    assert bool((got[:, :col0] == 0x55).all()) and bool((got[:, col0 + n:] == 0x55).all())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("batch,seq,n,k", [(1, 200, 264, 384), (2, 256, 512, 256), (3, 512, 128, 128)])
def test_gemm_with_gate_and_residual_equals_the_two_kernels(ops, dtype, batch, seq, n, k):
    """lyraq_gemm_fp8_gate = lyraq_gemm_fp8 followed by lyraq_gate_residual, bit for bit (the same roundings in the same
    order), also in place on the residual."""
    m = batch * seq
    w = workloads.fp8_linear(m=m, k=k, n=n, seed=m + n, dtype=dtype)
    g = torch.Generator().manual_seed(n)
    gate = torch.randn(batch, n, generator=g).to(dtype)
    res = torch.randn(m, n, generator=g).to(dtype)
    y = torch.empty(m, n, dtype=dtype, device="cuda")
    ops.gemm_with_residual_and_bias_fp8(cu(w["qw"]), cu(w["s_w"]), cu(w["qx"]), cu(w["s_x"]), y, bias=cu(w["bias"]))
    want = torch.empty(batch, seq, n, dtype=dtype, device="cuda")
    ops.invoke_fused_gate_and_residual(want, y.view(batch, seq, n), cu(gate), cu(res).view(batch, seq, n))
    got = torch.empty(m, n, dtype=dtype, device="cuda")
    assert ops.gemm_fp8_gate_residual(cu(w["qw"]), cu(w["s_w"]), cu(w["qx"]), cu(w["s_x"]), got, cu(gate), cu(res), seq,
                                      bias=cu(w["bias"]))
    check_status()
    assert_bit_equal(got, want.view(m, n).cpu())
    inplace = cu(res).clone()
    ops.gemm_fp8_gate_residual(cu(w["qw"]), cu(w["s_w"]), cu(w["qx"]), cu(w["s_x"]), inplace, cu(gate), inplace, seq, bias=cu(w["bias"]))
    assert_bit_equal(inplace, want.view(m, n).cpu())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,heads,k,tile", [(200, 2, 256, 0), (512, 3, 384, 0), (700, 4, 3072, 0), (300, 2, 256, 2561), (520, 4, 2048, 2562)])
def test_qkv_gemm_with_fused_qk_norm_and_rope_equals_the_two_kernels(ops, dtype, m, heads, k, tile):
    """lyraq_gemm_fp8_qk_rope = lyraq_gemm_fp8 followed by lyraq_rmsnorm_rope in place, bit for bit (the same roundings and the
    same order of the fp32 sums), with one CTA per tile and with CTA pairs, into a plain output and into a row window of a
    taller tensor (the joint sequence of a double-stream block); v heads and the rows around the window are untouched."""
    from lyradiff_b200 import _lib
    n = 3 * heads * 128
    w = workloads.fp8_linear(m=m, k=k, n=n, seed=m + heads, dtype=dtype)
    g = torch.Generator().manual_seed(m)
    scale = (1.0 + 0.2 * torch.randn(2 * 128, generator=g)).to(dtype)
    ang = torch.rand(m, 64, generator=g) * 6.28
    rope = torch.stack([torch.cos(ang), -torch.sin(ang), torch.sin(ang), torch.cos(ang)], dim=-1).to(dtype)
    want = torch.empty(m, n, dtype=dtype, device="cuda")
    ops.gemm_with_residual_and_bias_fp8(cu(w["qw"]), cu(w["s_w"]), cu(w["qx"]), cu(w["s_x"]), want, bias=cu(w["bias"]))
    plain = want.clone()
    ops.invoke_fused_rmsnorm_and_rope(want, want, cu(scale), cu(rope), 1e-6, 1, m, heads, 128)
    assert _lib.lib().lyraq_debug_force_gemm_tile(tile) == 0
    try:
        got = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
        ops.gemm_fp8_qk_rope(cu(w["qw"]), cu(w["s_w"]), cu(w["qx"]), cu(w["s_x"]), got, cu(scale), cu(rope), heads, 128, bias=cu(w["bias"]))
        tall = torch.full((m + 37, n), 3.0, dtype=dtype, device="cuda")
        ops.gemm_fp8_qk_rope(cu(w["qw"]), cu(w["s_w"]), cu(w["qx"]), cu(w["s_x"]), tall[16:16 + m], cu(scale), cu(rope), heads, 128,
                             bias=cu(w["bias"]))
    finally:
        _lib.lib().lyraq_debug_force_gemm_tile(0)
    check_status()
    assert_bit_equal(got, want.cpu())
    assert_bit_equal(got[:, 2 * heads * 128:], plain[:, 2 * heads * 128:].cpu(), "v heads")
    assert not torch.equal(got[:, :2 * heads * 128], plain[:, :2 * heads * 128])
    assert_bit_equal(tall[16:16 + m], want.cpu(), "row window")
    assert bool((tall[:16] == 3.0).all()) and bool((tall[16 + m:] == 3.0).all())


def test_fused_qk_rope_gemm_refuses_other_head_sizes(ops):
    from lyradiff_b200 import _lib
    p = 0x10000
    L = _lib.lib()
    assert L.lyraq_gemm_fp8_qk_rope(p, p, p, p, p, 192, 1, None, p, p, 1, 64, 1e-6, 128, 192, 128, None) == 2   # LYRAQ_ERR_UNSUPPORTED
    assert L.lyraq_gemm_fp8_qk_rope(p, p, p, p, p, 768, 1, None, p, p, 1, 128, 1e-6, 128, 768, 128, None) == 2  # n != 3 * heads * 128
    assert L.lyraq_gemm_fp8_qk_rope(p, p, p, p, p, 384, 2, None, p, p, 1, 128, 1e-6, 128, 384, 128, None) == 1  # fp32 output: invalid


def test_gate_fusion_refuses_tiles_that_straddle_batches(ops):
    w = workloads.fp8_linear(m=200, k=128, n=128, seed=1)
    y = torch.empty(200, 128, dtype=torch.bfloat16, device="cuda")
    gate = torch.ones(2, 128, dtype=torch.bfloat16, device="cuda")
    assert ops.gemm_fp8_gate_residual(cu(w["qw"]), cu(w["s_w"]), cu(w["qx"]), cu(w["s_x"]), y, gate, y, 100) is False


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n", [8, 1000, 3072 * 64 + 5])
@pytest.mark.parametrize("alpha", [1.0, 0.3])
def test_load_lora_rounds_like_the_16_bit_operators(dt, n, alpha):
    from lyradiff_b200 import ops
    from oracle import quant
    g = torch.Generator().manual_seed(n)
    w = torch.randn(n, generator=g).to(dt)
    lora = (torch.randn(n, generator=g) * 0.05).to(dt)
    got = cu(w).clone()
    ops.invoke_load_lora(got, cu(lora), alpha)
    assert_bit_equal(got, quant.load_lora(w, lora, alpha), "load_lora")
    check_status()
