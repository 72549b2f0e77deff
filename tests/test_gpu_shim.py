"""Runs include/lyradiff_shim.h: every reference-named function is called with the reference's own argument order
(tests/shim_runner.cpp, one exported wrapper per call form) on real device buffers, and its result must equal, bit for
bit, the same operation issued through lyradiff_b200.ops (the C ABI directly), which the oracle tests cover."""

import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

from tests.util import assert_bit_equal, check_status, cu

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "shim_runner.cpp")
OUT = os.path.join(ROOT, "tests", "_build", "libshim_runner.so")


def _build():
    deps = [SRC, os.path.join(ROOT, "include", "lyradiff_shim.h"), os.path.join(ROOT, "include", "lyraq.h")]
    if os.path.exists(OUT) and all(os.path.getmtime(d) <= os.path.getmtime(OUT) for d in deps):
        return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    libdir = os.path.join(ROOT, "lyradiff_b200")
    cmd = ["g++", "-std=c++17", "-O1", "-fPIC", "-shared", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
           SRC, "-o", OUT, "-L", libdir, "-llyraq", "-L", os.path.join(cuda, "lib64"), "-lcudart", "-Wl,-rpath," + libdir]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return OUT


@pytest.fixture(scope="module")
def shim():
    from lyradiff_b200 import _lib
    _lib.lib()                                   # liblyraq.so first, so that the runner binds to the same copy
    lib = ctypes.CDLL(_build())
    lib.shim_last_error.restype = ctypes.c_char_p

    def call(name, *args):
        conv = []
        for a in args:
            if isinstance(a, torch.Tensor):
                assert a.is_cuda and a.is_contiguous()
                conv.append(ctypes.c_void_p(a.data_ptr()))
            elif a is None:
                conv.append(ctypes.c_void_p(0))
            elif isinstance(a, float):
                conv.append(a)                   # wrapped by the caller as c_float / c_double
            elif isinstance(a, (bytes,)):
                conv.append(ctypes.c_char_p(a))
            elif isinstance(a, int):
                conv.append(ctypes.c_size_t(a))
            else:
                conv.append(a)
        rc = getattr(lib, name)(*conv)
        assert rc == 0, lib.shim_last_error().decode()
    call.lib = lib
    return call


@pytest.fixture(scope="module")
def ops():
    from lyradiff_b200 import ops as _ops
    return _ops


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


I = ctypes.c_int
F = ctypes.c_float
D = ctypes.c_double


def test_sdxl_int8_forms(shim, ops):
    g = torch.Generator().manual_seed(1)
    batch, seq, dim = 2, 96, 640
    x = cu(torch.randn(batch, seq, dim, generator=g).half())
    pre = cu(0.5 + torch.rand(dim, generator=g))
    s1 = cu(torch.tensor([0.05]))
    s_tok = cu(0.02 + 0.05 * torch.rand(batch * seq, generator=g))
    for per_token, s in ((0, s1), (1, s_tok)):
        a = torch.empty(batch, seq, dim, dtype=torch.int8, device="cuda")
        b = torch.empty_like(a)
        shim("shim_sq_input_quant", a, x, pre, s, I(per_token), batch, seq, dim, _stream())
        ops.invoke_sq_input_quant(b, x, pre, s, per_token=bool(per_token))
        assert_bit_equal(a, b.cpu(), "invokeSqInputQuant per_token=%d" % per_token)

    gamma, beta = cu((1 + 0.1 * torch.randn(dim, generator=g)).half()), cu((0.1 * torch.randn(dim, generator=g)).half())
    a, b = (torch.empty(batch, seq, dim, dtype=torch.int8, device="cuda") for _ in range(2))
    shim("shim_layer_norm_int8o", a, x, gamma, beta, pre, s1, batch, seq, dim, _stream(), D(1e-5))
    ops.invoke_layer_norm_int8o(b, x, gamma, beta, pre, s1, eps=1e-5)
    assert_bit_equal(a, b.cpu(), "invokeLayerNormInt8O")

    res = cu(torch.randn(batch, seq, dim, generator=g).half())
    bias = cu((0.1 * torch.randn(dim, generator=g)).half())
    a2, b2 = (torch.empty(batch, seq, dim, dtype=torch.float16, device="cuda") for _ in range(2))
    shim("shim_residual_bias_layer_norm_int8o", a, a2, x, res, bias, gamma, beta, pre, s1, batch, seq, dim, _stream(), D(1e-5))
    ops.invoke_layer_norm_int8o(b, x, gamma, beta, pre, s1, eps=1e-5, residual=res, bias=bias, sum_out=b2)
    assert_bit_equal(a, b.cpu(), "invokeFusedResidualBiasLayerNormInt8O int8")
    assert_bit_equal(a2, b2.cpu(), "invokeFusedResidualBiasLayerNormInt8O sum")

    inner = 256
    h = cu(torch.randn(batch, seq, 2 * inner, generator=g).half())
    hb = cu((0.1 * torch.randn(2 * inner, generator=g)).half())
    pre2 = cu(0.5 + torch.rand(inner, generator=g))
    for v2 in (0, 1):
        a, b = (torch.empty(batch, seq, inner, dtype=torch.int8, device="cuda") for _ in range(2))
        shim("shim_add_bias_geglu_int8o", a, h, hb, pre2, s1, I(seq), I(inner), I(batch), _stream(), I(v2))
        ops.invoke_fused_add_bias_geglu_int8o(b, h, hb, pre2, s1)
        assert_bit_equal(a, b.cpu(), "invokeFusedAddBiasGegluInt8O v2=%d" % v2)

    n, k, m = 320, dim, batch * seq
    w = cu((torch.randn(n, k, generator=g) * 0.02).half())
    qa, qb = (torch.empty(n, k, dtype=torch.int8, device="cuda") for _ in range(2))
    sa, sb = (torch.empty(n, dtype=torch.float32, device="cuda") for _ in range(2))
    shim("shim_get_int8_weight_scale", sa, qa, w, pre, n, k, _stream())
    ops.invoke_get_int8_weight_scale(sb, qb, w, pre)
    assert_bit_equal(qa, qb.cpu(), "invokeGetINT8WeightScale q")
    assert_bit_equal(sa, sb.cpu(), "invokeGetINT8WeightScale scale")

    act = torch.empty(m, k, dtype=torch.int8, device="cuda")
    ops.invoke_sq_input_quant(act, x, pre, s1)
    for per_token, s in ((0, s1), (1, s_tok)):
        ya, yb = (torch.empty(m, n, dtype=torch.float16, device="cuda") for _ in range(2))
        shim("shim_run_gemm_int8", act, qa, sa, s, ya, I(m), I(n), I(k), None, _stream(), I(per_token))
        ops.run_gemm_int8(act, qb, sb, s, yb, per_token=bool(per_token))
        assert_bit_equal(ya, yb.cpu(), "runGemmInt8 per_token=%d" % per_token)
    gb = cu((0.05 * torch.randn(n, generator=g)).half())
    r = cu(torch.randn(m, n, generator=g).half())
    ya, yb = (torch.empty(m, n, dtype=torch.float16, device="cuda") for _ in range(2))
    shim("shim_run_gemm_int8_bias_residual", act, qa, sa, s1, ya, gb, r, I(m), I(n), I(k), _stream())
    ops.run_gemm_int8(act, qb, sb, s1, yb, bias=gb, residual=r)
    assert_bit_equal(ya, yb.cpu(), "runGemmInt8BiasResidual")
    check_status()


def test_flux_fp8_forms(shim, ops):
    g = torch.Generator().manual_seed(2)
    batch, seq, dim, n = 2, 160, 512, 384
    m = batch * seq
    x = cu(torch.randn(batch, seq, dim, generator=g).bfloat16())
    s = cu(torch.tensor([0.02]))
    a, b = (torch.empty(m, dim, dtype=torch.uint8, device="cuda") for _ in range(2))
    shim("shim_d2d_scale_cpy_convert", a, x, s, I(1), m * dim, _stream())
    ops.invoke_cuda_d2d_scale_cpy_convert(b, x, s)
    assert_bit_equal(a, b.cpu(), "invokeCudaD2DScaleCpyConvert")

    w = cu((torch.randn(n, dim, generator=g) * 0.02).bfloat16())
    sa, sb = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    shim("shim_get_fp8_weight_scale", sa, w, n * dim, _stream())
    ops.invoke_get_fp8_weight_scale(sb, w)
    assert_bit_equal(sa, sb.cpu(), "invokeGetFP8WeightScale")

    wa, wb = w.clone(), w.clone()
    lora = cu((torch.randn(n, dim, generator=g) * 0.01).bfloat16())
    shim("shim_load_lora", wa, lora, n * dim, F(0.7), _stream())
    ops.invoke_load_lora(wb, lora, 0.7)
    assert_bit_equal(wa, wb.cpu(), "invokeLoadLora")

    sc, sh = cu((0.1 * torch.randn(batch, dim, generator=g)).bfloat16()), cu((0.1 * torch.randn(batch, dim, generator=g)).bfloat16())
    ya, yb = torch.empty_like(x), torch.empty_like(x)
    shim("shim_layer_norm_shift_scale", ya, x, sc, sh, batch, seq, dim, _stream())
    ops.invoke_layer_norm_with_shift_and_scale(yb, x, sc, sh, eps=1e-6)
    assert_bit_equal(ya, yb.cpu(), "invokeLayerNormWithShiftAndScale")
    shim("shim_layer_norm_shift_scale_fp8o", a, s, ya, x, sc, sh, batch, seq, dim, _stream())
    ops.invoke_layer_norm_with_shift_and_scale(yb, x, sc, sh, eps=1e-6, qf8=b, f8_scale=s)
    assert_bit_equal(a, b.cpu(), "invokeLayerNormWithShiftAndScaleFp8O e4m3")
    assert_bit_equal(ya, yb.cpu(), "invokeLayerNormWithShiftAndScaleFp8O y")

    heads, hd = 2, 128
    qkv = cu(torch.randn(batch, seq, 3 * heads * hd, generator=g).bfloat16())
    qs = cu((1 + 0.1 * torch.randn(2 * hd, generator=g)).bfloat16())
    ang = torch.rand(m, hd // 2, generator=g) * 6.28
    rope = cu(torch.stack([torch.cos(ang), -torch.sin(ang), torch.sin(ang), torch.cos(ang)], dim=-1).bfloat16())
    ra, rb = torch.empty_like(qkv), torch.empty_like(qkv)
    shim("shim_rmsnorm_rope", ra, qkv, qs, rope, F(1e-6), I(batch), I(seq), I(heads), I(hd), _stream())
    ops.invoke_fused_rmsnorm_and_rope(rb, qkv, qs, rope, 1e-6, batch, seq, heads, hd)
    assert_bit_equal(ra, rb.cpu(), "invokeFusedRmsNormAndRope")

    gate = cu(torch.randn(batch, dim, generator=g).bfloat16())
    res = cu(torch.randn(batch, seq, dim, generator=g).bfloat16())
    shim("shim_gate_residual", ya, x, gate, res, I(batch), I(seq), I(dim), _stream())
    ops.invoke_fused_gate_and_residual(yb, x, gate, res)
    assert_bit_equal(ya, yb.cpu(), "invokeFusedGateAndResidual")

    qw = torch.empty(n, dim, dtype=torch.uint8, device="cuda")
    ops.invoke_cuda_d2d_scale_cpy_convert(qw, w, sb)
    bias = cu((0.02 * torch.randn(n, generator=g)).bfloat16())
    r2 = cu(torch.randn(m, n, generator=g).bfloat16())
    for is_gelu, resid, beta in ((0, None, 0.0), (1, None, 0.0), (0, r2, 1.0)):
        ga, gb = (torch.empty(m, n, dtype=torch.bfloat16, device="cuda") for _ in range(2))
        shim("shim_gemm_fp8", I(n), I(m), I(dim), qw, sb, b, s, ga, bias, resid, F(1.0), F(beta), I(is_gelu), _stream(), I(0))
        ops.gemm_with_residual_and_bias_fp8(qw, sb, b, s, gb, bias=bias, residual=resid, alpha=1.0, beta=beta, is_gelu=bool(is_gelu))
        assert_bit_equal(ga, gb.cpu(), "GemmWithResidualAndBias gelu=%d residual=%s" % (is_gelu, resid is not None))
    # any other layout is refused with an exception, as documented
    rc = shim.lib.shim_gemm_fp8(n, m, dim, ctypes.c_void_p(qw.data_ptr()), ctypes.c_void_p(sb.data_ptr()), ctypes.c_void_p(b.data_ptr()),
                                ctypes.c_void_p(s.data_ptr()), ctypes.c_void_p(ga.data_ptr()), None, None, F(1.0), F(0.0), 0, _stream(), 1)
    assert rc == 1 and b"OP_T" in shim.lib.shim_last_error()
    check_status()


def test_flux_w4a4_forms_and_weight_container(shim, ops, tmp_path):
    g = torch.Generator().manual_seed(3)
    m, k, n = 256, 256, 384
    x = cu(torch.randn(m, k, generator=g).bfloat16())
    smooth = cu(0.5 + torch.rand(k, generator=g))
    down = cu((torch.randn(32, k, generator=g) * 0.05).bfloat16())
    up = cu((torch.randn(n, 32, generator=g) * 0.05).bfloat16())
    w = cu((torch.randn(n, k, generator=g) * 0.02).bfloat16())
    qw = torch.empty(n, k // 2, dtype=torch.uint8, device="cuda")
    sw = torch.empty(n, k // 64, dtype=torch.float32, device="cuda")
    ops.weight_quant_int4_g64(qw, sw, w)

    qa, qb = (torch.empty(m, k // 2, dtype=torch.uint8, device="cuda") for _ in range(2))
    ssa, ssb = (torch.empty(m, k // 64, dtype=torch.float32, device="cuda") for _ in range(2))
    ca, cb = (torch.empty(m, 32, dtype=torch.float32, device="cuda") for _ in range(2))
    shim("shim_quantize_lora_down", ca, qa, ssa, x, down, smooth, I(m), I(32), I(k), I(k // 64), _stream())
    ops.invoke_fused_quantize_and_lora_down_simple(cb, qb, ssb, x, down, smooth)
    assert_bit_equal(qa, qb.cpu(), "invokeFusedQuantizeAndLoraDownSimple q")
    assert_bit_equal(ssa, ssb.cpu(), "invokeFusedQuantizeAndLoraDownSimple scales")
    assert_bit_equal(ca, cb.cpu(), "invokeFusedQuantizeAndLoraDownSimple act")

    act16 = ca.bfloat16()                       # the reference converts the fp32 activation to T between the two calls
    da, db = (torch.empty(m, n, dtype=torch.bfloat16, device="cuda") for _ in range(2))
    shim("shim_w4a4_gemm_lora_up", da, qa, qw, act16, up, ssa, sw, I(m), I(n), I(k), I(32), I(k // 64), _stream())
    ops.invoke_fused_w4a4_gemm_and_lora_up(db, qb, qw, act16, up, ssb, sw)
    assert_bit_equal(da, db.cpu(), "invokeFusedW4A4GemmAndLoraUp")

    # W4A4GemmWeight<T>::loadWeights from the reference's .bin files (16-bit tensors stored as fp32 and as fp16 files),
    # then W4A4Gemm<T>::forward == lyraq_w4a4_lora_forward on the same tensors
    from lyradiff_b200 import layers
    lin = layers.W4A4Gemm(qw, sw, smooth=smooth, lora_down=down, lora_up=up)
    want = lin.forward(x)
    for file_type, np_dt in ((0, np.float32), (1, np.float16)):
        prefix = str(tmp_path / ("t%d_" % file_type))
        qw.cpu().numpy().tofile(prefix + "packed_weight.bin")
        sw.cpu().numpy().tofile(prefix + "weight_scale.bin")
        smooth.cpu().numpy().tofile(prefix + "smooth.bin")
        # values that survive the file type: take them from the device tensors, store, and compare against a layer built
        # from what the file holds
        up_f, down_f = up.cpu().float().numpy().astype(np_dt), down.cpu().float().numpy().astype(np_dt)
        up_f.tofile(prefix + "lora_up.bin")
        down_f.tofile(prefix + "lora_down.bin")
        if file_type == 0:
            ref = want
        else:
            lin16 = layers.W4A4Gemm(qw, sw, smooth=smooth, lora_down=cu(torch.from_numpy(down_f.astype(np.float32)).bfloat16()),
                                    lora_up=cu(torch.from_numpy(up_f.astype(np.float32)).bfloat16()))
            ref = lin16.forward(x)
        got = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        shim("shim_w4a4_layer_from_bins", got, x, m, n, k, prefix.encode(), I(file_type), _stream())
        assert_bit_equal(got, ref.cpu(), "W4A4Gemm::forward from .bin files (type %d)" % file_type)
    check_status()
