"""Activation and weight quantizers of the reference, restated on the CPU (test infrastructure).

All arithmetic is IEEE fp32 with round-half-to-even, as the reference's device
code defines it; the reference's release build adds --use_fast_math
(CMakeLists.txt:69,187-188), whose approximate divide is deliberately not
imitated.  Tensors are torch CPU tensors; integer outputs are int8 / uint8 /
int32 torch tensors.
"""

import numpy as np
import torch

from . import e4m3 as _e4m3

F32 = torch.float32


def _f32(x):
    return x.to(F32)


def _rne_sat(v, lo, hi):
    """cvt.rni.sat: round-half-to-even then clamp; NaN converts to 0 like the PTX cvt."""
    v = torch.nan_to_num(v, nan=0.0, posinf=float(hi), neginf=float(lo))
    return torch.clamp(torch.round(v), lo, hi)


# --------------------------------------------------------------------------- INT8 activations
def sq_input_quant(x, pre_quant_scale, input_quant_scale, per_token=False):
    """SmoothQuant activation quantize with a given scale.

    Follows sqInputQuant / sqPerTokenInputQuant
    (src/lyradiff/kernels/quant_kernels/quant_kernels.cu:51-115) and
    float_to_int8_rn (src/lyradiff/kernels/quant_kernels/int8_utils.cuh:23-28):
    q = sat_s8(rne((float(x) * pre[c]) / s)), s = scalar or s[row]; range [-128, 127].
    x: [rows, dim]; pre_quant_scale: fp32 [dim] or None (== ones).
    """
    v = _f32(x)
    if pre_quant_scale is not None:
        v = v * _f32(pre_quant_scale)[None, :]
    s = _f32(input_quant_scale).reshape(-1)
    s = s[:, None] if per_token else s[0]
    return _rne_sat(v / s, -128, 127).to(torch.int8)


def dynamic_per_token_scale(x, pre_quant_scale):
    """Per-token dynamic scale s[row] = max_c |float(x)*pre[c]| / 127 (fp32 divide); all-zero row -> 1.

    Not in the reference (its per-token kernel takes precomputed scales,
    quant_kernels.cu:93-115); this is the dynamic variant the SDXL GEGLU-FF
    configuration asks for, defined with the reference's own operand order.
    """
    v = _f32(x)
    if pre_quant_scale is not None:
        v = v * _f32(pre_quant_scale)[None, :]
    amax = torch.nan_to_num(v.abs(), nan=0.0).amax(dim=1)   # a maximum taken with fmaxf drops NaN operands
    s = amax / torch.tensor(127.0, dtype=F32)
    return torch.where(amax == 0, torch.ones_like(s), s)


def sq_input_quant_dynamic(x, pre_quant_scale):
    s = dynamic_per_token_scale(x, pre_quant_scale)
    return sq_input_quant(x, pre_quant_scale, s, per_token=True), s


def smooth_vector(x, w, alpha=0.5):
    """SmoothQuant smoothing vector s_j = max|X_j|^alpha / max|W_j|^(1-alpha) (configuration 1's rule)."""
    ax = _f32(x).abs().amax(dim=0)
    aw = _f32(w).abs().amax(dim=0)
    return (ax.pow(alpha) / aw.pow(1.0 - alpha)).to(F32)


# --------------------------------------------------------------------------- INT8 weights
def int8_weight_quant_device(w, pre_quant_scale):
    """Load-time per-output-channel weight quantize, device twin.

    Follows GetINT8WeightScale (quant_kernels.cu:173-223): w' = float(w) / pre[c];
    s_w[n] = float(double(amax_n) / 127.0); q = sat_s8(rne(w' / s_w)) in [-128, 127].
    An all-zero row gives s_w = 0 and 0/0 = NaN, which cvt converts to 0.
    """
    v = _f32(w)
    if pre_quant_scale is not None:
        v = v / _f32(pre_quant_scale)[None, :]
    amax = v.abs().amax(dim=1)
    s = (amax.double() / 127.0).to(F32)
    q = _rne_sat(v / s[:, None], -128, 127).to(torch.int8)
    return q, s


def int8_weight_quant_offline(w_folded):
    """Offline exporter's rule (lyradiff/convert_model_scripts/convert_sd_quant_model.py:108-155):
    q = clamp(rne(W' * (127/amax_n)), -127, 127), s_w = amax_n/127; amax <= 2**-24 -> q = 0, s_w = 1."""
    v = _f32(w_folded)
    amax = v.abs().amax(dim=1)
    tiny = amax <= 2.0 ** -24
    scale = torch.tensor(127.0, dtype=F32) / amax
    q = torch.clamp(torch.round(v * scale[:, None]), -127, 127)
    q = torch.where(tiny[:, None], torch.zeros_like(q), q).to(torch.int8)
    s = torch.where(tiny, torch.ones_like(amax), amax / torch.tensor(127.0, dtype=F32))
    return q, s


# --------------------------------------------------------------------------- FP8 e4m3
def fp8_quant(x, scale, invert_scale=True):
    """Per-tensor static-scale e4m3 quantize.

    Follows cudaD2DScaleCpyConvert (src/lyradiff/utils/memory_utils.cu:431-439):
    r = 1.0f / scale[0] when invert_scale else scale[0]; q = e4m3_rne_satfinite(float(x) * r).
    Returns uint8 codes.
    """
    s = _f32(scale).reshape(-1)[0]
    r = (torch.tensor(1.0, dtype=F32) / s) if invert_scale else s
    v = (_f32(x) * r).numpy()
    return torch.from_numpy(_e4m3.encode(v))


def fp8_amax_scale(w, prev=None):
    """scale = max(prev, max|w| / 448), follows getFP8WeightScale (src/lyradiff/kernels/lora/load_lora.cu:49-54)."""
    s = (_f32(w).abs() / torch.tensor(448.0, dtype=F32)).amax().reshape(1)
    if prev is not None:
        s = torch.maximum(s, _f32(prev).reshape(1))
    return s


def fp8_dequant(bits):
    return torch.from_numpy(_e4m3.decode(bits.numpy()))


# --------------------------------------------------------------------------- INT4, group 64
def pack_int4(q):
    """int values in [-8, 7], shape [rows, K] -> uint8 [rows, K/2], element 2i in the low nibble.

    Layout of fused_quantized_and_lora_down_simple's output
    (src/lyradiff/kernels/w4a4_gemm/w4a4_gemm.cu:206-214,914-929): eight nibbles per
    32-bit word, element 8j+i at bits 4i, which in little-endian bytes is exactly
    "even element in the low nibble of byte i/2".
    """
    qn = q.to(torch.int16).numpy() & 0xF
    lo = qn[:, 0::2]
    hi = qn[:, 1::2]
    return torch.from_numpy((lo | (hi << 4)).astype(np.uint8))


def unpack_int4(packed):
    p = packed.numpy().astype(np.int16)
    lo = p & 0xF
    hi = (p >> 4) & 0xF
    out = np.empty((p.shape[0], p.shape[1] * 2), dtype=np.int16)
    out[:, 0::2] = lo
    out[:, 1::2] = hi
    out = np.where(out >= 8, out - 16, out)
    return torch.from_numpy(out.astype(np.int8))


def int4_quant_g64(x, smooth, group=64):
    """Activation int4 quantize per (row, group of 64 columns).

    Follows w4a4_gemm.cu:897-930: v = float(x) / smooth[c]; s = max|v| / 7.0f;
    q = sat_s4(rne(v / s)).  An all-zero group gives s = 0 and v/s = NaN, which the
    reference's cvt.rni.s32.f32 turns into 0; the same is done here (s = 0, q = 0).
    Returns (packed uint8 [M, K/2], scales fp32 [M, K/group], unpacked int8 [M, K]).
    """
    v = _f32(x)
    if smooth is not None:
        v = v / _f32(smooth)[None, :]
    m, k = v.shape
    vg = v.reshape(m, k // group, group)
    s = torch.nan_to_num(vg.abs(), nan=0.0).amax(dim=2) / torch.tensor(7.0, dtype=F32)   # fmaxf drops NaN operands
    q = _rne_sat(vg / s[:, :, None], -8, 7).reshape(m, k).to(torch.int8)
    return pack_int4(q), s.contiguous(), q


def int4_weight_quant_g64(w, group=64):
    """Weight int4 quantize per (output channel, group of 64 along K).

    The reference has no weight quantizer for this format
    (lyradiff/convert_model_scripts/convert_flux_w4a4_bin.py only dumps tensors); the rule is
    defined symmetric to the activation rule, with the packed layout the kernel reads
    (src/lyradiff/layers/w4a4_gemm_block/W4A4GemmWeight.h:21): [N, K/2] bytes, even k low.
    """
    return int4_quant_g64(w, None, group)


def lora_down(x, down):
    """Low-rank down projection computed next to the int4 quantize by fused_quantized_and_lora_down_simple
    (src/lyradiff/kernels/w4a4_gemm/w4a4_gemm.cu:769-954): act[m, r] = sum_k x[m, k] * down[r, k] on the
    UNSMOOTHED 16-bit x, fp32 result.  The reference adds its 64-column partial sums with floating-point atomics in
    no fixed order; the oracle sums in fp64 and rounds once, which every order agrees with to a few fp32 ulps."""
    return (x.double() @ down.double().t()).to(F32)


def load_lora(w, lora, alpha):
    """LoRA merge into a 16-bit weight, loadLora<T> (src/lyradiff/kernels/lora/load_lora.cu:6-14):
    dst += src * T(alpha) with T's own operators, i.e. the product and the sum each rounded to T."""
    dt = w.dtype
    a = torch.tensor(alpha, dtype=F32).to(dt)
    t = (lora.to(F32) * a.to(F32)).to(dt)
    return (w.to(F32) + t.to(F32)).to(dt)
