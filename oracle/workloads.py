"""Seeded synthetic inputs with the shapes and distributions of the benchmark configurations
(test infrastructure).  They stand in for real SDXL / FLUX activations and calibrated scales,
which are not available offline.  Everything is generated on the CPU in fp32 from one
torch.Generator, in a fixed order, then cast, so every machine sees identical bits.
"""

import torch

from . import quant as _q

F32 = torch.float32


def _gen(seed):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def int8_smoothquant_linear(m=8192, k=640, n=5120, seed=0, dtype=torch.float16):
    """SDXL GEGLU-FF shaped INT8 SmoothQuant linear: X ~ N(0,1) with 5% of channels x20,
    W ~ N(0,0.02), bias ~ N(0,0.02); smoothing vector, per-channel weight quant of the folded
    weight, per-token dynamic activation quant."""
    g = _gen(seed)
    x = torch.randn(m, k, generator=g, dtype=F32)
    n_out = max(1, (k * 5) // 100)
    cols = torch.randperm(k, generator=g)[:n_out]
    x[:, cols] *= 20.0
    w = torch.randn(n, k, generator=g, dtype=F32) * 0.02
    bias = torch.randn(n, generator=g, dtype=F32) * 0.02
    x, w, bias = x.to(dtype), w.to(dtype), bias.to(dtype)
    smooth = _q.smooth_vector(x, w)
    pre = (torch.tensor(1.0, dtype=F32) / smooth).to(F32)  # activation side multiplies by 1/s
    # weight side: W' = W * s = W / pre, per output channel symmetric int8
    qw, s_w = _q.int8_weight_quant_device(w, pre)
    return {"x": x, "w": w, "bias": bias, "smooth": smooth, "pre": pre, "qw": qw, "s_w": s_w}


def fp8_linear(m, k, n, seed=0, dtype=torch.bfloat16, with_bias=True, with_residual=False):
    """FLUX-shaped FP8 linear: X ~ N(0,1), W ~ N(0,0.02), per-tensor amax/448 scales."""
    g = _gen(seed)
    x = torch.randn(m, k, generator=g, dtype=F32).to(dtype)
    w = (torch.randn(n, k, generator=g, dtype=F32) * 0.02).to(dtype)
    out = {"x": x, "w": w}
    out["bias"] = (torch.randn(n, generator=g, dtype=F32) * 0.02).to(dtype) if with_bias else None
    out["residual"] = torch.randn(m, n, generator=g, dtype=F32).to(dtype) if with_residual else None
    out["s_x"] = _q.fp8_amax_scale(x)
    out["s_w"] = _q.fp8_amax_scale(w)
    out["qx"] = _q.fp8_quant(x, out["s_x"])
    out["qw"] = _q.fp8_quant(w, out["s_w"])
    return out


FLUX_FP8_LINEARS = (
    # name, K, N, gelu, residual
    ("qkv", 3072, 9216, False, False),
    ("out_proj", 3072, 3072, False, False),
    ("mlp_up_gelu", 3072, 12288, True, False),
    ("mlp_down_residual", 12288, 3072, False, True),
)
FLUX_TOKENS = 4608


def w4a4_linear(m=4608, k=3072, n=21504, seed=0, dtype=torch.bfloat16, smooth_nontrivial=False,
                scale_dtype=torch.float16):
    """FLUX single-block fused W4A4 linear: X ~ N(0,1), W ~ N(0,0.02), int4 group-64 both sides."""
    g = _gen(seed)
    x = torch.randn(m, k, generator=g, dtype=F32).to(dtype)
    w = (torch.randn(n, k, generator=g, dtype=F32) * 0.02).to(dtype)
    if smooth_nontrivial:
        smooth = (0.5 + torch.rand(k, generator=g, dtype=F32)).to(F32)
    else:
        smooth = torch.ones(k, dtype=F32)
    pw, sw, qw = _q.int4_weight_quant_g64(w)
    sw = sw.to(scale_dtype)
    return {"x": x, "w": w, "smooth": smooth, "packed_w": pw, "s_w": sw, "qw": qw}


def adaln_input(b=1, s=4608, d=3072, seed=0, dtype=torch.bfloat16):
    """AdaLN + quantize input: X ~ N(0,1); scale, shift ~ N(0,0.1) per batch row."""
    g = _gen(seed)
    x = torch.randn(b, s, d, generator=g, dtype=F32).to(dtype)
    scale = (torch.randn(b, d, generator=g, dtype=F32) * 0.1).to(dtype)
    shift = (torch.randn(b, d, generator=g, dtype=F32) * 0.1).to(dtype)
    return {"x": x, "scale": scale, "shift": shift}
