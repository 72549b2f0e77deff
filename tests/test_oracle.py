"""CPU tests of the oracle: known-answer facts of the number formats, exactness of the integer
contraction, and agreement with the committed golden vectors."""

import numpy as np
import torch

from oracle import e4m3, gemm, norms, quant, workloads


def test_e4m3_code_table_round_trip():
    codes = np.arange(256, dtype=np.uint8)
    vals = e4m3.decode(codes)
    finite = ~np.isnan(vals)
    assert finite.sum() == 254 and np.isnan(vals[0x7F]) and np.isnan(vals[0xFF])
    assert vals[0x7E] == 448.0 and vals[0xFE] == -448.0
    assert vals[0x01] == 2.0 ** -9 and vals[0x08] == 2.0 ** -6 and vals[0x38] == 1.0
    assert np.array_equal(e4m3.encode(vals[finite]), codes[finite])


def test_e4m3_rounding_and_saturation():
    x = np.array([448, 449, 464, 1e9, -1e9, 2.0 ** -10, 2.0 ** -10 * 1.01, 1.0625, 1.1875, 3 * 2.0 ** -10], dtype=np.float32)
    # ties go to the even mantissa; anything above 448 saturates (never NaN)
    assert e4m3.encode(x).tolist() == [0x7E, 0x7E, 0x7E, 0x7E, 0xFE, 0x00, 0x01, 0x38, 0x3A, 0x02]
    assert e4m3.encode(np.array([np.nan], dtype=np.float32))[0] == 0x7F


def test_e4m3_matches_torch_cast_after_clamp():
    g = torch.Generator().manual_seed(1)
    for scale in (1e-3, 1.0, 100.0):
        x = torch.randn(20000, generator=g) * scale
        ref = x.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        assert np.array_equal(e4m3.encode(x.numpy()), ref)


def test_int8_round_half_even_and_saturation():
    x = torch.tensor([[0.5, 1.5, 2.5, -0.5, -1.5, 127.4, 127.5, 300.0, -128.5, -129.0, -300.0, 0.0]], dtype=torch.float16)
    x = torch.cat([x, torch.zeros(1, 4, dtype=torch.float16)], dim=1)
    q = quant.sq_input_quant(x, None, torch.tensor([1.0]))
    assert q[0, :12].tolist() == [0, 2, 2, 0, -2, 127, 127, 127, -128, -128, -128, 0]


def test_int4_pack_layout_and_zero_group():
    q = torch.arange(-8, 8, dtype=torch.int8).repeat(1, 4)  # [1, 64]
    packed = quant.pack_int4(q)
    assert packed.shape == (1, 32)
    assert packed[0, 0].item() == ((-8) & 0xF) | (((-7) & 0xF) << 4)
    assert torch.equal(quant.unpack_int4(packed), q)
    x = torch.zeros(2, 128, dtype=torch.bfloat16)
    x[1, :64] = torch.linspace(-3, 3, 64).bfloat16()
    p, s, qi = quant.int4_quant_g64(x, None)
    assert s[0].tolist() == [0.0, 0.0] and int(qi[0].abs().sum()) == 0  # all-zero group: q = 0, s = 0
    assert qi[1, :64].min().item() == -7 and qi[1, :64].max().item() == 7


def test_int_matmul_exact_vs_int64():
    g = torch.Generator().manual_seed(2)
    a = torch.randint(-128, 128, (33, 3072), generator=g, dtype=torch.int8)
    b = torch.randint(-128, 128, (17, 3072), generator=g, dtype=torch.int8)
    ref = a.to(torch.int64) @ b.to(torch.int64).t()
    assert torch.equal(gemm.int_matmul_exact(a, b).to(torch.int64), ref)


def test_w4a4_unit_scales_is_exact_integer_sum():
    g = torch.Generator().manual_seed(3)
    qa = torch.randint(-8, 8, (16, 256), generator=g, dtype=torch.int8)
    qw = torch.randint(-8, 8, (24, 256), generator=g, dtype=torch.int8)
    y = gemm.w4a4_gemm(qa, qw, torch.ones(16, 4), torch.ones(24, 4), out_dtype=torch.float32)
    assert torch.equal(y.to(torch.int64), qa.to(torch.int64) @ qw.to(torch.int64).t())


def test_golden_int8(golden):
    z = golden("int8")
    qa, sa = quant.sq_input_quant_dynamic(z["x"], z["pre"])
    assert torch.equal(qa, z["qa"]) and torch.equal(sa, z["sa"])
    assert torch.equal(quant.sq_input_quant(z["x"], z["pre"], z["static_scale"]), z["q_static"])
    qw, s_w = quant.int8_weight_quant_device(z["w"], z["pre"])
    assert torch.equal(qw, z["qw"]) and torch.equal(s_w, z["s_w"])
    acc = gemm.int8_gemm_acc(qa, qw)
    assert torch.equal(acc, z["acc"])
    y = gemm.int8_gemm(qa, qw, s_w, sa, torch.float16, per_token=True, bias=z["bias"])
    assert torch.equal(y.view(torch.int16), z["y"].view(torch.int16))


def test_golden_fp8(golden):
    z = golden("fp8")
    assert torch.equal(quant.fp8_quant(z["x"], z["s_x"]), z["qx"])
    assert torch.equal(quant.fp8_amax_scale(z["w"]), z["s_w"])
    for key, kw in (("y_plain", {}), ("y_gelu", {"gelu": True}), ("y_residual", {"residual": z["residual"]})):
        y = gemm.fp8_gemm(z["qx"], z["qw"], z["s_x"], z["s_w"], bias=z["bias"], **kw)
        assert torch.equal(y.view(torch.int16), z[key].view(torch.int16))


def test_golden_w4a4(golden):
    z = golden("w4a4")
    pa, sa, qa = quant.int4_quant_g64(z["x"], z["smooth"])
    assert torch.equal(pa, z["packed_a"]) and torch.equal(sa, z["sa"])
    pw, sw, qw = quant.int4_weight_quant_g64(z["w"])
    assert torch.equal(pw, z["packed_w"]) and torch.equal(sw, z["s_w"])
    assert torch.equal(gemm.w4a4_gemm(qa, qw, sa, sw, out_dtype=torch.float32), z["y_f32"])


def test_golden_adaln_and_ln(golden):
    z = golden("adaln")
    o = norms.adaln_quant(z["x"], z["scale"], z["shift"], fp8_scale=z["f8_scale"])
    assert torch.equal(o["q8"], z["q8"]) and torch.equal(o["s8"], z["s8"]) and torch.equal(o["qf8"], z["qf8"])
    assert torch.equal(o["y"].view(torch.int16), z["y"].view(torch.int16))
    z = golden("ln_geglu")
    q, _ = norms.layernorm_int8(z["x"], z["gamma"], z["beta"], z["pre"], z["scale"])
    assert torch.equal(q, z["q_ln"])
    q, h = norms.layernorm_int8(z["x"], z["gamma"], z["beta"], z["pre"], z["scale"], residual=z["residual"], bias=z["bias"])
    assert torch.equal(q, z["q_rln"]) and torch.equal(h.view(torch.int16), z["hsum"].view(torch.int16))
    assert torch.equal(norms.geglu_int8(z["h"], z["b2"], z["pre"], z["scale"]), z["q_geglu"])


def test_adaln_matches_plain_fp32_layernorm_within_bf16():
    a = workloads.adaln_input(b=2, s=16, d=256, seed=5)
    y = norms.adaln_modulate(a["x"], a["scale"], a["shift"]).float()
    x = a["x"].float()
    ref = torch.nn.functional.layer_norm(x, (256,), eps=1e-6) * (1 + a["scale"].float()[:, None]) + a["shift"].float()[:, None]
    assert (y - ref).abs().max() < 0.05


def test_smoothquant_linear_accuracy_small():
    wl = workloads.int8_smoothquant_linear(m=64, k=640, n=32, seed=0)
    qa, sa = quant.sq_input_quant_dynamic(wl["x"], wl["pre"])
    y = gemm.int8_gemm(qa, wl["qw"], wl["s_w"], sa, torch.float16, per_token=True, bias=wl["bias"]).float()
    ref = wl["x"].float() @ wl["w"].float().t() + wl["bias"].float()
    assert ((y - ref).norm() / ref.norm()).item() < 0.03
