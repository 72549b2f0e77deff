"""CPU restatement of the FLUX blocks (FP8 single- and double-stream, INT4 single-stream), for the parity tests of
lyradiff_b200.flux_blocks.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  PARITY UNPINNED: the reference has no test or golden vector for
this block; the data flow follows FluxSingleTransformerFP8Block<T>::forward
(src/lyradiff/layers/flux_single_transformer_block/FluxSingleTransformerFP8Block.cc:162-310), AdaFP8LayerNorm<T>::forward
(src/lyradiff/layers/ada_layer_norm/AdaFP8LayerNorm.cc:96-205) and FluxSingleAttentionFP8Processor<T>::forward
(src/lyradiff/layers/flux_single_attention_processor/FluxSingleAttentionFP8Processor.cc:134-230), with the kernels'
arithmetic restated in oracle/quant.py, gemm.py and norms.py and an exact (fp64) softmax attention.
"""

import torch

from . import gemm as _g
from . import norms as _n
from . import quant as _q

F32 = torch.float32


def _fp8_linear(x, w, bias, s_x, out_dtype, gelu=False, cache=None, key=None):
    """Quantize-on-load weight (per-tensor amax / 448), static activation scale, FP8 GEMM.  `cache` keeps the quantized
    weight between calls, as the loaded layer does."""
    if cache is not None and key in cache:
        qw, s_w = cache[key]
    else:
        s_w = _q.fp8_amax_scale(w)
        qw = _q.fp8_quant(w, s_w)
        if cache is not None:
            cache[key] = (qw, s_w)
    return _g.fp8_gemm(_q.fp8_quant(x, s_x), qw, s_x, s_w, out_dtype=out_dtype, bias=bias, gelu=gelu)


def attention(q, k, v):
    """softmax(q k^T / sqrt(d)) v per head in fp64; q, k, v [B, H, S, Dh]."""
    d = q.shape[-1]
    p = torch.softmax(q.double() @ k.double().transpose(-1, -2) / (d ** 0.5), dim=-1)
    return p @ v.double()


def flux_single_block(hidden, rope, temb, sd, prefix, heads, head_dim, mlp_scale=4, quant_level=1, cache=None):
    """hidden [B, S, D], rope [B, S, head_dim/2, 2, 2], temb [B, D] (SiLU'd); sd: the state dict the block loads;
    cache: optional dict that keeps the quantized weights between calls.  Returns (out [B, S, D], intermediates)."""
    dt = hidden.dtype
    B, S, D = hidden.shape
    g = lambda name: sd[prefix + name]
    if quant_level == 2:
        msa = _fp8_linear(temb, g("norm.linear.weight").to(dt), g("norm.linear.bias").to(dt), g("norm.linear_input_scale"), dt, cache=cache, key="norm")
    else:
        msa = (temb.double() @ g("norm.linear.weight").to(dt).double().t() + g("norm.linear.bias").to(dt).double()).to(dt)
    shift, scale, gate = msa.chunk(3, dim=1)
    norm = _n.adaln_modulate(hidden, scale, shift, eps=1e-6)                                  # [B, S, D] of dt
    n2 = norm.reshape(B * S, D)
    qkv = _fp8_linear(n2, g("attn.to_qkv.weight").to(dt), g("attn.to_qkv.bias").to(dt), g("attn.to_qkv_input_scale"), dt, cache=cache, key="qkv")
    qk_scale = torch.cat([g("attn.norm_q.weight").reshape(-1), g("attn.norm_k.weight").reshape(-1)]).to(dt)
    qkv = _n.rmsnorm_rope(qkv, qk_scale, rope.reshape(B * S, head_dim // 2, 2, 2), heads, head_dim, eps=1e-6)
    v5 = qkv.reshape(B, S, 3, heads, head_dim)
    q, k, v = (v5[:, :, i].transpose(1, 2) for i in range(3))
    attn = attention(q, k, v).transpose(1, 2).reshape(B * S, D).to(dt)
    mlp = _fp8_linear(n2, g("proj_mlp.weight").to(dt), g("proj_mlp.bias").to(dt), g("proj_mlp_input_scale"), dt, gelu=True, cache=cache, key="mlp")
    cat = torch.cat([attn, mlp], dim=1)
    y = _fp8_linear(cat, g("proj_out.weight").to(dt), g("proj_out.bias").to(dt), g("proj_out_input_scale"), dt, cache=cache, key="out")
    out = _n.gate_residual(y.reshape(B, S, D), gate, hidden)
    return out, {"msa": msa, "norm": norm, "qkv": qkv, "attn": attn, "mlp": mlp, "y": y}


def flux_double_block(hidden, encoder, rope, temb, sd, prefix, heads, head_dim, quant_level=1, cache=None):
    """Double-stream block: FluxTransformerFP8Block<T>::forward
    (src/lyradiff/layers/flux_transformer_block/FluxTransformerFP8Block.cc:155-245) with FluxAttentionFP8Processor
    (layers/flux_attention_processor/FluxAttentionFP8Processor.cc:140-340) and FluxAttnPostFP8Processor
    (layers/flux_attn_post_processor/FluxAttnPostFP8Processor.cc:90-205).  hidden [B, S, D] (image), encoder [B, E, D]
    (text), rope [B, E + S, head_dim/2, 2, 2] over the joint sequence with the text first.  Returns (hidden_out, encoder_out)."""
    dt = hidden.dtype
    B, S, D = hidden.shape
    E = encoder.shape[1]
    g = lambda name: sd[prefix + name]
    cache = {} if cache is None else cache

    def lin(x, name, gelu=False):
        return _fp8_linear(x, g(name + ".weight").to(dt), g(name + ".bias").to(dt), g(name + "_input_scale"), dt, gelu=gelu,
                           cache=cache, key=name)

    def modulation(norm):
        if quant_level == 2:
            msa = lin(temb, norm + ".linear")
        else:
            msa = (temb.double() @ g(norm + ".linear.weight").to(dt).double().t() + g(norm + ".linear.bias").to(dt).double()).to(dt)
        return msa.chunk(6, dim=1)

    streams = {"img": (hidden, "norm1", "attn.to_qkv", "attn.to_out.0", "attn.norm_q.weight", "attn.norm_k.weight", "ff"),
               "txt": (encoder, "norm1_context", "attn.to_added_qkv", "attn.to_add_out", "attn.norm_added_q.weight",
                       "attn.norm_added_k.weight", "ff_context")}
    mods, qkvs = {}, {}
    rope_j = rope.reshape(B, E + S, head_dim // 2, 2, 2)
    for key, (x, norm, qkv_name, _, nq, nk, _) in streams.items():
        mod = modulation(norm)
        n = _n.adaln_modulate(x, mod[1], mod[0], eps=1e-6).reshape(-1, D)
        qkv = lin(n, qkv_name)
        scale = torch.cat([g(nq).reshape(-1), g(nk).reshape(-1)]).to(dt)
        L = x.shape[1]
        r = (rope_j[:, :E] if key == "txt" else rope_j[:, E:]).reshape(B * L, head_dim // 2, 2, 2)
        qkvs[key] = _n.rmsnorm_rope(qkv, scale, r, heads, head_dim, eps=1e-6).reshape(B, L, 3 * D)
        mods[key] = mod
    joint = torch.cat([qkvs["txt"], qkvs["img"]], dim=1).reshape(B, E + S, 3, heads, head_dim)
    q, k, v = (joint[:, :, i].transpose(1, 2) for i in range(3))
    attn = attention(q, k, v).transpose(1, 2).reshape(B, E + S, D).to(dt)
    outs = {}
    for key, (x, _, _, out_name, _, _, ff) in streams.items():
        mod = mods[key]
        a = (attn[:, :E] if key == "txt" else attn[:, E:]).reshape(-1, D)
        L = x.shape[1]
        y = lin(a, out_name).reshape(B, L, D)
        h = _n.gate_residual(y, mod[2], x)
        n2 = _n.adaln_modulate(h, mod[4], mod[3], eps=1e-6).reshape(-1, D)
        f1 = lin(n2, ff + ".net.0.proj", gelu=True)
        f2 = lin(f1, ff + ".net.2").reshape(B, L, D)
        outs[key] = _n.gate_residual(f2, mod[5], h)
    return outs["img"], outs["txt"]


def _w4a4_linear(x, sd, name, out_dtype, gelu=False, residual=None):
    """One W4A4 linear as W4A4Gemm<T>::forward runs it (src/lyradiff/layers/w4a4_gemm_block/W4A4Gemm.cc:113-169): int4
    quantize of x / smooth with the low-rank down projection beside it, grouped s4 GEMM + LoRA-up stored as T, then the
    reference's separate 16-bit kernels for bias / GELU / residual, each of which rounds to T (round_each).
    Weights under `name`: packed_weight uint8 [n, k/2], weight_scale [n, k/64], smooth fp32 [k], lora_down T [32, k],
    lora_up T [n, 32], optional bias T [n] (the file names of W4A4GemmWeight<T>::loadWeights, W4A4GemmWeight.cc:62-79)."""
    _, sa, qa = _q.int4_quant_g64(x, sd[name + "smooth"])
    act = _q.lora_down(x, sd[name + "lora_down"].to(out_dtype))
    qw = _q.unpack_int4(sd[name + "packed_weight"])
    return _g.w4a4_gemm(qa, qw, sa, sd[name + "weight_scale"], out_dtype=out_dtype, bias=sd.get(name + "bias"), gelu=gelu,
                        residual=residual, lora_act=act, lora_up=sd[name + "lora_up"].to(out_dtype), round_each=True)


def flux_single_block_int4(hidden, rope, temb, sd, prefix, heads, head_dim, mlp_scale=4, quant_level=7):
    """INT4 single-stream block: FluxSingleTransformerInt4Block<T>::forward
    (src/lyradiff/layers/flux_single_transformer_block/FluxSingleTransformerInt4Block.cc:198-322) with
    FluxSingleAttentionInt4Processor<T>::forward
    (src/lyradiff/layers/flux_single_attention_processor/FluxSingleAttentionInt4Processor.cc:138-192).
    quant_level 7: 16-bit modulation linear; 8: FP8 modulation linear.  proj_out is two W4A4 linears, one over the
    attention output (with the bias) and one over the MLP activation, summed by fusedBiasAndResidual."""
    dt = hidden.dtype
    B, S, D = hidden.shape
    g = lambda name: sd[prefix + name]
    if quant_level == 8:
        msa = _fp8_linear(temb, g("norm.linear.weight").to(dt), g("norm.linear.bias").to(dt), g("norm.linear_input_scale"), dt)
    else:
        msa = (temb.double() @ g("norm.linear.weight").to(dt).double().t() + g("norm.linear.bias").to(dt).double()).to(dt)
    shift, scale, gate = msa.chunk(3, dim=1)
    n2 = _n.adaln_modulate(hidden, scale, shift, eps=1e-6).reshape(B * S, D)
    qkv = _w4a4_linear(n2, sd, prefix + "attn.to_qkv.", dt)  # the bias add of fuseBiasRmsNormAndRope is the T-rounded step
    qk_scale = torch.cat([g("attn.norm_q.weight").reshape(-1), g("attn.norm_k.weight").reshape(-1)]).to(dt)
    qkv = _n.rmsnorm_rope(qkv, qk_scale, rope.reshape(B * S, head_dim // 2, 2, 2), heads, head_dim, eps=1e-6)
    v5 = qkv.reshape(B, S, 3, heads, head_dim)
    q, k, v = (v5[:, :, i].transpose(1, 2) for i in range(3))
    attn = attention(q, k, v).transpose(1, 2).reshape(B * S, D).to(dt)
    mlp = _w4a4_linear(n2, sd, prefix + "proj_mlp.", dt, gelu=True)
    h1 = _w4a4_linear(attn, sd, prefix + "proj_out.linears.0.", dt)
    h = _w4a4_linear(mlp, sd, prefix + "proj_out.linears.1.linear.", dt, residual=h1)
    out = _n.gate_residual(h.reshape(B, S, D), gate, hidden)
    return out, {"msa": msa, "qkv": qkv, "attn": attn, "mlp": mlp, "h": h}


def flux_double_block_int4(hidden, encoder, rope, temb, sd, prefix, heads, head_dim, quant_level=7):
    """INT4 double-stream block: FluxTransformerInt4Block<T>::forward
    (src/lyradiff/layers/flux_transformer_block/FluxTransformerInt4Block.cc:155-240) with
    FluxAttentionInt4Processor<T>::forward (layers/flux_attention_processor/FluxAttentionInt4Processor.cc:157-305) and
    FluxAttnPostInt4Processor<T>::forward (layers/flux_attn_post_processor/FluxAttnPostInt4Processor.cc).  Per stream:
    16-bit AdaLN, W4A4 to_qkv (+ invokeAddBias), joint QK norm / RoPE / attention, W4A4 to_out (+ invokeAddBias), gate +
    residual, 16-bit AdaLN, W4A4 net.0.proj (+ invokeFusedBiasAndGelu), e4m3 quantize, FP8 net.2, gate + residual."""
    dt = hidden.dtype
    B, S, D = hidden.shape
    E = encoder.shape[1]
    g = lambda name: sd[prefix + name]
    cache = {}

    def modulation(norm):
        if quant_level == 8:
            msa = _fp8_linear(temb, g(norm + ".linear.weight").to(dt), g(norm + ".linear.bias").to(dt),
                              g(norm + ".linear_input_scale"), dt)
        else:
            msa = (temb.double() @ g(norm + ".linear.weight").to(dt).double().t() + g(norm + ".linear.bias").to(dt).double()).to(dt)
        return msa.chunk(6, dim=1)

    streams = {"img": (hidden, "norm1", "attn.to_qkv.", "attn.to_out.0.", "attn.norm_q.weight", "attn.norm_k.weight", "ff"),
               "txt": (encoder, "norm1_context", "attn.to_added_qkv.", "attn.to_add_out.", "attn.norm_added_q.weight",
                       "attn.norm_added_k.weight", "ff_context")}
    mods, qkvs = {}, {}
    rope_j = rope.reshape(B, E + S, head_dim // 2, 2, 2)
    for key, (x, norm, qkv_name, _, nq, nk, _) in streams.items():
        mod = modulation(norm)
        n = _n.adaln_modulate(x, mod[1], mod[0], eps=1e-6).reshape(-1, D)
        qkv = _w4a4_linear(n, sd, prefix + qkv_name, dt)
        scale = torch.cat([g(nq).reshape(-1), g(nk).reshape(-1)]).to(dt)
        L = x.shape[1]
        r = (rope_j[:, :E] if key == "txt" else rope_j[:, E:]).reshape(B * L, head_dim // 2, 2, 2)
        qkvs[key] = _n.rmsnorm_rope(qkv, scale, r, heads, head_dim, eps=1e-6).reshape(B, L, 3 * D)
        mods[key] = mod
    joint = torch.cat([qkvs["txt"], qkvs["img"]], dim=1).reshape(B, E + S, 3, heads, head_dim)
    q, k, v = (joint[:, :, i].transpose(1, 2) for i in range(3))
    attn = attention(q, k, v).transpose(1, 2).reshape(B, E + S, D).to(dt)
    outs = {}
    for key, (x, _, _, out_name, _, _, ff) in streams.items():
        mod = mods[key]
        a = (attn[:, :E] if key == "txt" else attn[:, E:]).reshape(-1, D)
        L = x.shape[1]
        ao = _w4a4_linear(a, sd, prefix + out_name, dt).reshape(B, L, D)
        h = _n.gate_residual(ao, mod[2], x)
        n2 = _n.adaln_modulate(h, mod[4], mod[3], eps=1e-6).reshape(-1, D)
        f1 = _w4a4_linear(n2, sd, prefix + ff + ".net.0.proj.", dt, gelu=True)
        name = ff + ".net.2"
        f2 = _fp8_linear(f1, g(name + ".weight").to(dt), g(name + ".bias").to(dt), g(name + "_input_scale"), dt, cache=cache,
                         key=name).reshape(B, L, D)
        outs[key] = _n.gate_residual(f2, mod[5], h)
    return outs["img"], outs["txt"]
