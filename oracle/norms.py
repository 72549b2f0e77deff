"""LayerNorm / AdaLN / GEGLU producers that feed the quantizers, restated on the CPU (test infrastructure).

Row statistics are computed in fp64 and rounded to fp32 (the reference keeps
Welford state in fp32 for AdaLN and in half for the int8 LayerNorm; neither
summation order is reproducible, so the oracle states the exact value and the
tests allow the documented 1-LSB slack on a small fraction of outputs).
Everything after the statistics follows the reference's rounding sequence
exactly: each arithmetic step in the tensor type T is rounded to T.
"""

import torch

from . import quant as _q

F32 = torch.float32


def _row_stats(x, eps):
    xd = x.double()
    mean = xd.mean(dim=-1, keepdim=True)
    var = ((xd - mean) ** 2).mean(dim=-1, keepdim=True).clamp_min(0.0)
    rstd = 1.0 / torch.sqrt(var + eps)
    return mean.to(F32), rstd.to(F32)


def _t(v, dtype):
    """Round an fp32 intermediate to the tensor type and bring it back (one T-precision op)."""
    return v.to(dtype).to(F32)


def adaln_modulate(x, scale, shift, eps=1e-6):
    """AdaLN-Zero modulation y = LN(x) * (1 + scale_b) + shift_b, no affine.

    Follows LayerNormBlockWithShiftAndScaleSMemImpl (src/lyradiff/kernels/norms/layer_norm.cu:405-484):
    fp32 statistics (population variance clamped at 0, rsqrt(var + eps)); x_hat rounded to T;
    then (scale + 1) * x_hat + shift evaluated in T arithmetic with each of the three
    operations rounded to T.  x: [B, S, D] of T; scale, shift: [B, D] of T.
    """
    dt = x.dtype
    mean, rstd = _row_stats(x, eps)
    xhat = _t((x.to(F32) - mean) * rstd, dt)
    sp1 = _t(scale.to(F32) + 1.0, dt)[:, None, :]
    prod = _t(sp1 * xhat, dt)
    y = _t(prod + shift.to(F32)[:, None, :], dt)
    return y.to(dt)


def adaln_quant(x, scale, shift, eps=1e-6, fp8_scale=None, pre_quant_scale=None):
    """Fused AdaLN-modulate + quantize: what the reference does as two kernels
    (layer_norm.cu:405-484, then memory_utils.cu:431-446 or quant_kernels.cu:93-115).

    Returns dict with y (T), q8/int8 + s8 (dynamic per-token scale) and, if fp8_scale is given,
    qf8 (e4m3 codes, static per-tensor scale).
    """
    y = adaln_modulate(x, scale, shift, eps)
    b, s, d = y.shape
    y2 = y.reshape(b * s, d)
    q8, s8 = _q.sq_input_quant_dynamic(y2, pre_quant_scale)
    out = {"y": y, "q8": q8, "s8": s8}
    if fp8_scale is not None:
        out["qf8"] = _q.fp8_quant(y2, fp8_scale, invert_scale=True)
    return out


def layernorm_affine(x, gamma, beta, eps=1e-5):
    """LayerNorm with affine in T arithmetic: x_hat = T((x-mean)*rstd); y = T(T(gamma*x_hat) + beta).

    Rounding sequence of warpLayerNormInt8O (src/lyradiff/kernels/quant_kernels/layer_norm_int8.cu:430-556),
    with exact statistics in place of its half-precision Welford state.
    """
    dt = x.dtype
    mean, rstd = _row_stats(x, eps)
    xhat = _t((x.to(F32) - mean) * rstd, dt)
    y = _t(_t(gamma.to(F32) * xhat, dt) + beta.to(F32), dt)
    return y.to(dt)


def layernorm_int8(x, gamma, beta, pre_quant_scale, input_quant_scale, eps=1e-5, residual=None, bias=None):
    """(residual + bias +) LayerNorm -> int8 with a static scalar scale.

    Follows invokeLayerNormInt8O / invokeFusedResidualBiasLayerNormInt8O
    (layer_norm_int8.cu:558-679; kernels :102-556).  With a residual the sum
    h = T(T(x + residual) + bias) is formed in T arithmetic first and is also returned.
    """
    dt = x.dtype
    h = x
    if residual is not None:
        hf = _t(x.to(F32) + residual.to(F32), dt)
        if bias is not None:
            hf = _t(hf + bias.to(F32), dt)
        h = hf.to(dt)
    y = layernorm_affine(h, gamma, beta, eps)
    q = _q.sq_input_quant(y, pre_quant_scale, input_quant_scale, per_token=False)
    return q, h


def gelu_half_reference(g, dt):
    """GeluActivation<half2> / <bf162> (src/lyradiff/kernels/activation_kernels.h:70-100):
    cube in T, tanh argument and cdf in fp32, cdf rounded to T, product in T."""
    gf = g.to(F32)
    cube = _t(gf * _t(gf * gf, dt), dt)
    cdf = 0.5 * (1.0 + torch.tanh(0.7978845608028654 * (gf + 0.044715 * cube)))
    return _t(gf * _t(cdf, dt), dt)


def geglu_int8(h, bias, pre_quant_scale, input_quant_scale):
    """bias + GEGLU(tanh-GELU) -> int8.

    Follows fusedAddBiasGegluInt8O (src/lyradiff/kernels/quant_kernels/ffn_kernels_int8.cu:102-147):
    input [rows, 2*dim]; hidden = T(h[:, :dim] + b[:dim]); gate = T(h[:, dim:] + b[dim:]);
    gate = gelu(gate) (T); q = sat_s8(rne(float(T(hidden*gate)) * pre[c] / s)).
    The device tanh is tanh.approx.f32, so parity is within 1 LSB on a small fraction.
    """
    dt = h.dtype
    dim = h.shape[1] // 2
    hf = h.to(F32)
    if bias is not None:
        bf = bias.to(F32)
        hid = _t(hf[:, :dim] + bf[:dim], dt)
        gate = _t(hf[:, dim:] + bf[dim:], dt)
    else:
        hid, gate = hf[:, :dim], hf[:, dim:]
    gate = gelu_half_reference(gate, dt)
    prod = _t(hid * gate, dt)
    return _q.sq_input_quant(prod, pre_quant_scale, input_quant_scale, per_token=False)


def rmsnorm_rope(qkv, scale, rope, heads, head_dim, eps=1e-6):
    """QK RMSNorm + rotary embedding on the packed QKV projection.

    Follows fuseRmsNormAndRope (src/lyradiff/kernels/rope/flux_apply_rope.cu:8-76).  qkv [tokens, 3*heads*head_dim]
    (q heads, k heads, v heads); scale [2*head_dim] (q then k); rope [tokens, head_dim/2, 2, 2].  Per q/k head:
    inv = rsqrt(mean(x^2) + eps) (exact here, rsqrtf on the device); t = T(x*inv); t = T(t*scale);
    out[2i]   = T(T(t[2i]*r[i,0,0]) + T(t[2i+1]*r[i,0,1]));
    out[2i+1] = T(T(t[2i]*r[i,1,0]) + T(t[2i+1]*r[i,1,1]));  v heads are copied.
    """
    dt = qkv.dtype
    tokens = qkv.shape[0]
    x = qkv.reshape(tokens, 3, heads, head_dim)
    out = x.clone()
    r = rope.reshape(tokens, head_dim // 2, 2, 2).to(F32)
    for part in range(2):  # q, k
        xf = x[:, part].to(F32)                                   # [tokens, heads, head_dim]
        ms = (xf.double() ** 2).mean(dim=-1, keepdim=True)
        inv = (1.0 / torch.sqrt(ms + eps)).to(F32)
        t = _t(xf * inv, dt)
        t = _t(t * scale[part * head_dim:(part + 1) * head_dim].to(F32)[None, None, :], dt)
        te, to = t[..., 0::2], t[..., 1::2]                       # [tokens, heads, head_dim/2]
        o_even = _t(_t(te * r[:, None, :, 0, 0], dt) + _t(to * r[:, None, :, 0, 1], dt), dt)
        o_odd = _t(_t(te * r[:, None, :, 1, 0], dt) + _t(to * r[:, None, :, 1, 1], dt), dt)
        o = torch.stack([o_even, o_odd], dim=-1).reshape(tokens, heads, head_dim)
        out[:, part] = o.to(dt)
    return out.reshape(tokens, 3 * heads * head_dim)


def gate_residual(y, gate, x):
    """fuseGateAndResidual (src/lyradiff/kernels/flux_single_transformer_block/flux_single_transformer_kernels.cu:43-65):
    out = T(T(y * gate[b]) + x), y and x [B, S, D], gate [B, D]."""
    dt = y.dtype
    return _t(_t(y.to(F32) * gate.to(F32)[:, None, :], dt) + x.to(F32), dt).to(dt)
