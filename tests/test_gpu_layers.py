"""GPU tests of the quantized-Linear layer forwards (quantize into caller workspace + GEMM in one C-ABI call):
bit-identical to calling the quantizer and the GEMM separately, and checked against the oracle chain."""

import pytest
import torch

from oracle import gemm, quant, workloads
from tests.util import assert_bit_equal, check_status, cu, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def layers():
    from lyradiff_b200 import layers as _layers
    return _layers


def test_fp8_linear_layer(layers):
    f = workloads.fp8_linear(300, 512, 392, seed=31, with_residual=True)
    lin = layers.Fp8Linear(cu(f["w"]), cu(f["bias"]), f["s_x"], gelu=False)
    assert torch.equal(lin.qweight.cpu(), f["qw"]) and torch.equal(lin.w_scale.cpu(), f["s_w"])
    y = lin.forward(cu(f["x"]), residual=cu(f["residual"]))
    want = gemm.fp8_gemm(f["qx"], f["qw"], f["s_x"], f["s_w"], bias=f["bias"], residual=f["residual"])
    assert rel_err(y, want) < 1e-2
    lin_g = layers.Fp8Linear(cu(f["w"]), cu(f["bias"]), f["s_x"], gelu=True)
    yg = lin_g.forward(cu(f["x"]).view(3, 100, 512))
    assert yg.shape == (3, 100, 392)
    assert rel_err(yg.view(300, 392), gemm.fp8_gemm(f["qx"], f["qw"], f["s_x"], f["s_w"], bias=f["bias"], gelu=True)) < 1e-2
    check_status()


def test_int8_linear_layer_dynamic_and_static(layers):
    wl = workloads.int8_smoothquant_linear(m=260, k=640, n=520, seed=32)
    lin = layers.SmoothQuantLinear.from_float(cu(wl["w"]), cu(wl["pre"]), bias=cu(wl["bias"]))
    assert torch.equal(lin.qweight.cpu(), wl["qw"])
    y = lin.forward(cu(wl["x"]))
    qa, sa = quant.sq_input_quant_dynamic(wl["x"], wl["pre"])
    assert_bit_equal(y, gemm.int8_gemm(qa, wl["qw"], wl["s_w"], sa, torch.float16, per_token=True, bias=wl["bias"]))
    s = torch.tensor([0.37], dtype=torch.float32)
    lin_s = layers.SmoothQuantLinear(cu(wl["qw"]), cu(wl["s_w"]), cu(wl["pre"]), bias=cu(wl["bias"]), input_scale=cu(s))
    ys = lin_s.forward(cu(wl["x"]))
    qs = quant.sq_input_quant(wl["x"], wl["pre"], s)
    assert_bit_equal(ys, gemm.int8_gemm(qs, wl["qw"], wl["s_w"], s, torch.float16, bias=wl["bias"]))
    check_status()


def test_w4a4_layer(layers):
    w = workloads.w4a4_linear(m=200, k=512, n=264, seed=33, smooth_nontrivial=True)
    g = torch.Generator().manual_seed(33)
    bias = (torch.randn(264, generator=g) * 0.1).bfloat16()
    res = torch.randn(200, 264, generator=g).bfloat16()
    lin = layers.W4A4Gemm.from_float(cu(w["w"]), smooth=cu(w["smooth"]), bias=cu(bias))
    assert torch.equal(lin.qweight.cpu(), w["packed_w"])
    y = lin.forward(cu(w["x"]), residual=cu(res))
    _, sa, qa = quant.int4_quant_g64(w["x"], w["smooth"])
    assert_bit_equal(y, gemm.w4a4_gemm(qa, w["qw"], sa, w["s_w"], bias=bias, residual=res))
    check_status()


def test_w4a4_layer_with_low_rank_branch(layers):
    """W4A4Gemm<T>::forward with lora_down / lora_up (W4A4Gemm.cc:137-163): compared with the oracle chain
    quantize -> down projection -> GEMM + up projection at one T ulp (the two low-rank sums are tensor-core fp32 sums)."""
    w = workloads.w4a4_linear(m=200, k=512, n=264, seed=34, smooth_nontrivial=True)
    g = torch.Generator().manual_seed(34)
    bias = (torch.randn(264, generator=g) * 0.1).bfloat16()
    down = (torch.randn(32, 512, generator=g) * 0.05).bfloat16()
    up = (torch.randn(264, 32, generator=g) * 0.2).bfloat16()
    lin = layers.W4A4Gemm.from_float(cu(w["w"]), smooth=cu(w["smooth"]), bias=cu(bias), lora_down=cu(down), lora_up=cu(up))
    y = lin.forward(cu(w["x"])).cpu()
    _, sa, qa = quant.int4_quant_g64(w["x"], w["smooth"])
    act = quant.lora_down(w["x"], down)
    want = gemm.w4a4_gemm(qa, w["qw"], sa, w["s_w"], bias=bias, lora_act=act, lora_up=up)
    plain = gemm.w4a4_gemm(qa, w["qw"], sa, w["s_w"], bias=bias)
    assert not torch.equal(want, plain)
    diff = (y.float() - want.float()).abs()
    bound = 2.0 ** -7 * want.float().abs() + 1e-3
    assert bool((diff <= bound).all()), float((diff / bound).max())
    assert float((diff > 0).float().mean()) <= 2e-2
    check_status()


def test_workspace_is_checked(layers):
    from lyradiff_b200 import _lib, ops
    L = _lib.lib()
    assert L.lyraq_workspace_bytes(4, 128, 256, 512) == 128 * 512
    assert L.lyraq_workspace_bytes(3, 100, 256, 640) == 100 * 640 + 512
    assert L.lyraq_workspace_bytes(5, 128, 256, 512) == 128 * 256 + 128 * 8 * 4
    x = torch.zeros(128, 512, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(256, 512, dtype=torch.uint8, device="cuda")
    y = torch.empty(128, 256, dtype=torch.bfloat16, device="cuda")
    s = torch.ones(1, device="cuda")
    small = torch.empty(1024, dtype=torch.uint8, device="cuda")
    st = L.lyraq_linear_fp8_forward(y.data_ptr(), x.data_ptr(), 1, s.data_ptr(), w.data_ptr(), s.data_ptr(), None, None, 0.0, 0,
                                    128, 256, 512, small.data_ptr(), small.numel(), None)
    assert st == 5  # LYRAQ_ERR_WORKSPACE


def test_int8_linear_from_the_reference_bin_layout(layers, tmp_path):
    """SDXL INT8 on-disk layout (<name>.weight_int8.bin, .weight_quant_scale.bin, .input_quant_scale.bin,
    .pre_quant_scale.bin, .bias.bin): write the files the exporter writes, read them back, same bits as the layer built
    from tensors; a short file is refused."""
    import numpy as np
    wl = workloads.int8_smoothquant_linear(m=130, k=640, n=200, seed=34)
    s = torch.tensor([0.21], dtype=torch.float32)
    prefix, name = str(tmp_path) + "/down_blocks.1.attentions.0.transformer_blocks.0.", "ff.net.0.proj"
    wl["qw"].numpy().tofile(prefix + name + ".weight_int8.bin")
    wl["s_w"].numpy().tofile(prefix + name + ".weight_quant_scale.bin")
    s.numpy().tofile(prefix + name + ".input_quant_scale.bin")
    wl["pre"].numpy().tofile(prefix + name + ".pre_quant_scale.bin")
    wl["bias"].numpy().astype(np.float16).tofile(prefix + name + ".bias.bin")
    lin = layers.SmoothQuantLinear.from_bin(prefix, name, 200, 640)
    ref = layers.SmoothQuantLinear(cu(wl["qw"]), cu(wl["s_w"]), cu(wl["pre"]), bias=cu(wl["bias"]), input_scale=cu(s))
    x = cu(wl["x"])
    assert_bit_equal(lin.forward(x), ref.forward(x).cpu())
    qs = quant.sq_input_quant(wl["x"], wl["pre"], s)
    assert_bit_equal(lin.forward(x), gemm.int8_gemm(qs, wl["qw"], wl["s_w"], s, torch.float16, bias=wl["bias"]))
    wl["s_w"].numpy()[:-1].tofile(prefix + name + ".weight_quant_scale.bin")
    with pytest.raises(RuntimeError, match="expected 200"):
        layers.SmoothQuantLinear.from_bin(prefix, name, 200, 640)
    check_status()
