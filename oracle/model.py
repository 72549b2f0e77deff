"""CPU restatement of the reference's whole FLUX transformer forward, for the parity test of lyradiff_b200.flux_model.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  PARITY UNPINNED: the reference has no test or golden vector for it.
Data flow of FluxTransformer2DModel<T>::transformer_forward
(src/lyradiff/models/flux_transformer_2d_model/FluxTransformer2DModel.cc:230-515); the quantized blocks are those of
oracle/blocks.py, the 16-bit linears around them are fp64 contractions rounded to T once (the reference's cuBLAS calls
accumulate in fp32 and add the bias before the one rounding).
"""

import math

import torch

from . import blocks as _b
from . import norms as _n

F32 = torch.float32


def time_projection(value, channels, dtype, max_period=10000.0):
    """TimeProjection<T>(channels, flip_sin_to_cos=true, downscale_freq_shift=0) (layers/time_proj/TimeProjection.cc:39-51;
    kernel kernels/time_proj/time_proj_kernels.cu:70-97): fp32 exponents exp(-ln(max_period) * i / half), fp32 sin / cos,
    cast to T, cosine half first."""
    half = channels // 2
    factor = torch.tensor(-math.log(max_period), dtype=F32) / half
    arg = torch.exp(factor * torch.arange(half, dtype=F32)) * torch.tensor(float(value), dtype=F32)
    return torch.cat([torch.cos(arg), torch.sin(arg)]).to(dtype).reshape(1, channels)


def _linear(x, w, b, dt):
    return (x.double() @ w.to(dt).double().t() + b.to(dt).double()).to(dt)


def _mlp(x, sd, prefix, dt):
    """TimestepEmbeddingBlock<T>::forward: Gemm -> T, fusedAddBiasSilu1D (T add, SiLU), GemmWithResidualAndBias."""
    h = (x.double() @ sd[prefix + "linear_1.weight"].to(dt).double().t()).to(dt)
    h = (h.to(F32) + sd[prefix + "linear_1.bias"].to(dt).to(F32)).to(dt)
    h = torch.nn.functional.silu(h.to(F32)).to(dt)
    return _linear(h, sd[prefix + "linear_2.weight"], sd[prefix + "linear_2.bias"], dt)


def flux_model(hidden, encoder, rope, pooled, timestep, guidance, sd, num_layers, num_single_layers, heads, head_dim,
               quant_level=1, controlnet_block_samples=None, controlnet_blocks_repeat=False):
    dt = hidden.dtype
    B, S, _ = hidden.shape
    E = encoder.shape[1]
    int4 = quant_level in (7, 8)
    t_emb = _mlp(time_projection(timestep, 256, dt), sd, "time_text_embed.timestep_embedder.", dt)
    g_emb = _mlp(time_projection(guidance, 256, dt), sd, "time_text_embed.guidance_embedder.", dt)
    p_emb = _mlp(pooled, sd, "time_text_embed.text_embedder.", dt)
    s = ((p_emb.to(F32) + g_emb.to(F32)).to(dt).to(F32) + t_emb.to(F32)).to(dt)        # add3Tensor2dAndSilu, T arithmetic
    temb = torch.nn.functional.silu(s.to(F32)).to(dt)
    h = _linear(hidden.reshape(B * S, -1), sd["x_embedder.weight"], sd["x_embedder.bias"], dt).reshape(B, S, -1)
    c = _linear(encoder.reshape(B * E, -1), sd["context_embedder.weight"], sd["context_embedder.bias"], dt).reshape(B, E, -1)
    samples = list(controlnet_block_samples or [])
    interval = (num_layers - 1) // len(samples) + 1 if samples else 0
    for i in range(num_layers):
        f = _b.flux_double_block_int4 if int4 else _b.flux_double_block
        h, c = f(h, c, rope, temb, sd, "transformer_blocks.%d." % i, heads, head_dim, quant_level)
        if samples:
            res = samples[i % len(samples)] if controlnet_blocks_repeat else samples[i // interval]
            h = (h.to(F32) + res.to(F32)).to(dt)
    x = torch.cat([c, h], dim=1)
    for j in range(num_single_layers):
        f = _b.flux_single_block_int4 if int4 else _b.flux_single_block
        x = f(x, rope, temb, sd, "single_transformer_blocks.%d." % j, heads, head_dim, 4, quant_level)[0]
    h = x[:, E:]
    msa = _linear(temb, sd["norm_out.linear.weight"], sd["norm_out.linear.bias"], dt)
    scale, shift = msa.chunk(2, dim=1)
    normed = _n.adaln_modulate(h, scale, shift, eps=1e-6)
    D = normed.shape[-1]
    return _linear(normed.reshape(B * S, D), sd["proj_out.weight"], sd["proj_out.bias"], dt).reshape(B, S, -1)
