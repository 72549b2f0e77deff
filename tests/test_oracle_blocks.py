"""CPU checks of the oracle's block-level functions against independent formulations (no GPU, no library)."""

import torch

from oracle import blocks, norms


def _rope(tokens, head_dim, g):
    ang = torch.rand(tokens, head_dim // 2, generator=g) * 6.28
    return torch.stack([torch.cos(ang), -torch.sin(ang), torch.sin(ang), torch.cos(ang)], dim=-1).reshape(tokens, head_dim // 2, 2, 2)


def test_rmsnorm_rope_is_a_rotation_of_the_normalised_head():
    g = torch.Generator().manual_seed(0)
    tokens, heads, hd = 6, 3, 128
    qkv = torch.randn(tokens, 3 * heads * hd, generator=g).bfloat16()
    scale = torch.ones(2 * hd).bfloat16()
    rope = _rope(tokens, hd, g)
    out = norms.rmsnorm_rope(qkv, scale, rope.bfloat16(), heads, hd, eps=1e-6).float().reshape(tokens, 3, heads, hd)
    x = qkv.float().reshape(tokens, 3, heads, hd)
    # v heads untouched
    assert torch.equal(out[:, 2], x[:, 2])
    # q, k: unit RMS after the norm, and a rotation keeps the length (bf16 rounding: 1 %)
    rms = out[:, :2].pow(2).mean(dim=-1).sqrt()
    assert float((rms - 1.0).abs().max()) < 0.02
    # against complex multiplication in fp32
    xn = x[:, :2] / x[:, :2].pow(2).mean(dim=-1, keepdim=True).sqrt()
    z = torch.complex(xn[..., 0::2], xn[..., 1::2])
    rot = torch.complex(rope[:, :, 0, 0], rope[:, :, 1, 0])[:, None, None, :]      # cos + i sin
    w = z * rot
    want = torch.stack([w.real, w.imag], dim=-1).reshape(tokens, 2, heads, hd)
    assert float((out[:, :2] - want).abs().max()) < 0.05


def test_gate_residual_rounds_after_each_step():
    y = torch.tensor([[[1.0078125, 3.0]]]).bfloat16()
    gate = torch.tensor([[1.0078125, 0.5]]).bfloat16()
    x = torch.tensor([[[0.00390625, 1.0]]]).bfloat16()
    out = norms.gate_residual(y, gate, x)
    # 1.0078125^2 = 1.01568... rounds to 1.015625 in bf16; + 2^-8 = 1.01953125 -> 1.0234375 or 1.015625 (tie to even)
    prod = torch.tensor(1.0078125 * 1.0078125).bfloat16().float()
    assert float(out[0, 0, 0]) == float((prod + 0.00390625).bfloat16())
    assert float(out[0, 0, 1]) == 2.5


def test_oracle_blocks_run_and_identity_gate_returns_the_input():
    g = torch.Generator().manual_seed(1)
    D, heads, hd = 256, 2, 128
    p = "b."
    sd = {}
    for name, n, k in (("norm.linear", 3 * D, D), ("attn.to_qkv", 3 * D, D), ("proj_mlp", 4 * D, D), ("proj_out", D, 5 * D)):
        sd[p + name + ".weight"] = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
        sd[p + name + ".bias"] = torch.zeros(n).bfloat16()
        sd[p + name + "_input_scale"] = torch.tensor([0.03])
    sd[p + "attn.norm_q.weight"] = torch.ones(hd).bfloat16()
    sd[p + "attn.norm_k.weight"] = torch.ones(hd).bfloat16()
    hidden = torch.randn(1, 24, D, generator=g).bfloat16()
    rope = _rope(24, hd, g).reshape(1, 24, hd // 2, 2, 2).bfloat16()
    temb = torch.randn(1, D, generator=g).bfloat16()
    out, mid = blocks.flux_single_block(hidden, rope, temb, sd, p, heads, hd, 4, 1)
    assert out.shape == hidden.shape and not torch.equal(out, hidden)
    assert set(mid) == {"msa", "norm", "qkv", "attn", "mlp", "y"}
    # a zero modulation linear gives gate = 0: the block returns its input
    sd[p + "norm.linear.weight"].zero_()
    out0, _ = blocks.flux_single_block(hidden, rope, temb, sd, p, heads, hd, 4, 1)
    assert torch.equal(out0, hidden)


def test_attention_matches_torch_sdpa():
    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn(1, 2, 17, 64, generator=g) for _ in range(3))
    want = torch.nn.functional.scaled_dot_product_attention(q, k, v)
    assert float((blocks.attention(q, k, v).float() - want).abs().max()) < 1e-5


def test_w4a4_round_each_differs_from_one_rounding_by_at_most_a_few_ulps():
    from oracle import gemm, quant
    g = torch.Generator().manual_seed(4)
    m, n, k = 24, 40, 128
    x = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    _, sw, qw = quant.int4_weight_quant_g64(w)
    _, sa, qa = quant.int4_quant_g64(x, None)
    bias = (torch.randn(n, generator=g) * 0.1).bfloat16()
    res = torch.randn(m, n, generator=g).bfloat16()
    once = gemm.w4a4_gemm(qa, qw, sa, sw, bias=bias, residual=res).float()
    each = gemm.w4a4_gemm(qa, qw, sa, sw, bias=bias, residual=res, round_each=True).float()
    # restated directly: three 16-bit kernels in a row
    acc = gemm.w4a4_gemm(qa, qw, sa, sw)                              # T(acc)
    step = (acc.float() + bias.float()).bfloat16()                    # add of two T values, rounded to T
    step = (step.float() + res.float()).bfloat16()
    assert torch.equal(each, step.float())
    # each of the two extra roundings moves the value by at most half a bf16 ulp of that step's magnitude
    mag = acc.float().abs() + bias.float().abs() + res.float().abs()
    assert bool(((each - once).abs() <= 2.0 ** -7 * mag).all())


def test_int4_block_oracle_zero_gate_returns_the_input():
    from oracle import quant
    g = torch.Generator().manual_seed(5)
    D, heads, hd, p = 128, 1, 128, "s."
    sd = {p + "norm.linear.weight": torch.zeros(3 * D, D).bfloat16(), p + "norm.linear.bias": torch.zeros(3 * D).bfloat16(),
          p + "attn.norm_q.weight": torch.ones(hd).bfloat16(), p + "attn.norm_k.weight": torch.ones(hd).bfloat16()}
    for name, n, k, bias in (("attn.to_qkv.", 3 * D, D, True), ("proj_mlp.", 4 * D, D, True), ("proj_out.linears.0.", D, D, True),
                             ("proj_out.linears.1.linear.", D, 4 * D, False)):
        pw, sw, _ = quant.int4_weight_quant_g64((torch.randn(n, k, generator=g) * 0.05).bfloat16())
        sd[p + name + "packed_weight"], sd[p + name + "weight_scale"] = pw, sw
        sd[p + name + "smooth"] = torch.ones(k)
        sd[p + name + "lora_down"] = (torch.randn(32, k, generator=g) * 0.02).bfloat16()
        sd[p + name + "lora_up"] = (torch.randn(n, 32, generator=g) * 0.05).bfloat16()
        if bias:
            sd[p + name + "bias"] = (torch.randn(n, generator=g) * 0.02).bfloat16()
    hidden = torch.randn(1, 12, D, generator=g).bfloat16()
    rope = _rope(12, hd, g).reshape(1, 12, hd // 2, 2, 2).bfloat16()
    temb = torch.randn(1, D, generator=g).bfloat16()
    out, mid = blocks.flux_single_block_int4(hidden, rope, temb, sd, p, heads, hd, 4, 7)
    assert torch.equal(out, hidden)                     # zero modulation linear -> gate 0 -> the residual alone
    assert float(mid["h"].float().abs().mean()) > 0.01  # while the branch itself is not zero
    sd[p + "norm.linear.bias"] = torch.cat([torch.zeros(2 * D), torch.ones(D)]).bfloat16()   # gate 1
    out1, mid1 = blocks.flux_single_block_int4(hidden, rope, temb, sd, p, heads, hd, 4, 7)
    assert torch.equal(out1, (mid1["h"].reshape(1, 12, D).float() + hidden.float()).bfloat16())


def test_time_projection_is_the_sinusoidal_embedding_with_the_cosine_half_first():
    import math
    from oracle import model
    e = model.time_projection(500.0, 256, torch.float32)
    assert tuple(e.shape) == (1, 256)
    # channel 0: frequency 1 -> cos(t), sin(t); the last channel: frequency max_period^-(127/128)
    assert abs(float(e[0, 0]) - math.cos(500.0)) < 1e-4 and abs(float(e[0, 128]) - math.sin(500.0)) < 1e-4
    w = math.exp(-math.log(10000.0) * 127 / 128)
    assert abs(float(e[0, 127]) - math.cos(500.0 * w)) < 1e-4 and abs(float(e[0, 255]) - math.sin(500.0 * w)) < 1e-4
    assert float((e[0, :128] ** 2 + e[0, 128:] ** 2 - 1.0).abs().max()) < 1e-5
