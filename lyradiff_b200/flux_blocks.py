"""Python mirror of the reference's block-level torch custom classes for the FLUX single-stream block.

`torch.classes.lyradiff.FluxSingleTransformerBlockOp` (src/lyradiff/th_op/pybind.cc:82-96,
th_op/flux_single_transformer_block/FluxSingleTransformerBlockOp.h:287-315) with the same constructor arguments,
method names and tensor conventions, running the FP8 data flow of FluxSingleTransformerFP8Block<T>::forward
(src/lyradiff/layers/flux_single_transformer_block/FluxSingleTransformerFP8Block.cc:162-310) on liblyraq.so:

    msa = linear(temb)                       -> shift, scale, gate            (temb arrives SiLU'd, AdaFP8LayerNorm.cc:100)
    norm = LN(x) * (1 + scale) + shift       -> bf16 and e4m3 in one kernel   (lyraq_adaln_quant)
    qkv = FP8 GEMM(norm_q8, to_qkv) + bias   -> QK RMSNorm + RoPE in place    (lyraq_gemm_fp8, lyraq_rmsnorm_rope)
    attn = attention(q, k, v)                                                 (torch SDPA: library code, as the reference's
                                                                              flash-attention layer is; not this path)
    cat8[:, :D]  = e4m3(attn)                                                 (lyraq_quant_fp8_2d)
    cat8[:, D:]  = e4m3(gelu(FP8 GEMM(e4m3(norm), proj_mlp) + bias))          (lyraq_quant_fp8, lyraq_gemm_fp8_quant_ld)
    y = FP8 GEMM(cat8, proj_out) + bias                                       (lyraq_gemm_fp8)
    out = gate * y + x                                                        (lyraq_gate_residual)

The 16-bit concat buffer and its quantize pass (invokeFusedCatAndGelu + invokeCudaD2DScaleCpyConvert) do not exist here.
quant_level 1 (FP8_W8A8) keeps the modulation linear in 16 bits (a torch matmul, as the reference calls cuBLAS for it),
quant_level 2 (FP8_W8A8_FULL) runs it in FP8 too.  Other levels, LoRA hot-swap and the .bin directory loader are not
built: they raise NotImplementedError.
"""

import torch

from . import ops

_DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16}
FP8_W8A8, FP8_W8A8_FULL = 1, 2


class LyraDiffCommonContext:
    """LyraDiffCommonContext (src/lyradiff/th_op/lyradiff_common_context/LyraDiffCommonContext.h:23-38): the reference's
    owner of stream, allocator and cuBLAS handles.  Here the kernels run on torch's current stream and buffers are torch
    tensors, so the context carries nothing."""

    def __init__(self):
        pass


class _Fp8Weight:
    """One quantized linear as MACROLoadFP8WeightFromCache leaves it (src/lyradiff/utils/common_macro_def.h:76-92)."""

    def __init__(self, weight, bias, input_scale, device, dtype):
        w = weight.to(device=device, dtype=dtype).contiguous()
        self.n, self.k = w.shape
        self.qweight = torch.empty(self.n, self.k, dtype=torch.uint8, device=device)
        self.w_scale = torch.empty(1, dtype=torch.float32, device=device)
        ops.weight_quant_fp8(self.qweight, self.w_scale, w)
        self.bias = None if bias is None else bias.to(device=device, dtype=dtype).contiguous()
        self.input_scale = input_scale.to(device=device, dtype=torch.float32).reshape(1).contiguous()


class FluxSingleTransformerBlockOp:
    def __init__(self, inference_dtype="bf16", embedding_dim=3072, embedding_head_num=24, embedding_head_dim=128, mlp_scale=4,
                 quant_level=0):
        if inference_dtype not in _DTYPES:
            raise RuntimeError("inference_dtype must be 'bf16' or 'fp16'")
        if quant_level not in (FP8_W8A8, FP8_W8A8_FULL):
            raise NotImplementedError("only quant_level 1 (FP8_W8A8) and 2 (FP8_W8A8_FULL) are built")
        if embedding_head_num * embedding_head_dim != embedding_dim:
            raise RuntimeError("embedding_dim must equal embedding_head_num * embedding_head_dim")
        self.dtype = _DTYPES[inference_dtype]
        self.dim, self.heads, self.head_dim, self.mlp_scale = embedding_dim, embedding_head_num, embedding_head_dim, mlp_scale
        self.quant_level = quant_level
        self._ctx = None
        self._w = None
        self._buf = {}

    # ---- reference method names (th_op/pybind.cc:82-96)
    def initialize(self, ctx):
        self._ctx = ctx

    def reload_model_from_bin(self, path, dtype):
        raise NotImplementedError("the .bin directory loader is not built; use reload_model_from_state_dict")

    def load_lora_by_name(self, names, weight, scale):
        raise NotImplementedError("LoRA hot-swap is not built")

    def clear_lora(self):
        raise NotImplementedError("LoRA hot-swap is not built")

    def reload_model_from_state_dict(self, prefix, state_dict, device):
        """Keys as the reference reads them (FluxSingleTransformerFP8BlockWeight.cc:135-149,
        FluxSingleAttentionFP8ProcessorWeight.cc:111-114): `<prefix>norm.linear.{weight,bias}`,
        `<prefix>attn.to_qkv.{weight,bias}`, `<prefix>attn.norm_q.weight`, `<prefix>attn.norm_k.weight`,
        `<prefix>proj_mlp.{weight,bias}`, `<prefix>proj_out.{weight,bias}` and the fp32 scalars
        `<prefix>attn.to_qkv_input_scale`, `<prefix>proj_mlp_input_scale`, `<prefix>proj_out_input_scale`
        (plus `<prefix>norm.linear_input_scale` at quant_level 2).  Host or device tensors; weights are quantized here."""
        dev = torch.device(device)
        sd = state_dict
        g = lambda name: sd[prefix + name]
        w = {}
        w["qkv"] = _Fp8Weight(g("attn.to_qkv.weight"), g("attn.to_qkv.bias"), g("attn.to_qkv_input_scale"), dev, self.dtype)
        w["mlp"] = _Fp8Weight(g("proj_mlp.weight"), g("proj_mlp.bias"), g("proj_mlp_input_scale"), dev, self.dtype)
        w["out"] = _Fp8Weight(g("proj_out.weight"), g("proj_out.bias"), g("proj_out_input_scale"), dev, self.dtype)
        if self.quant_level == FP8_W8A8_FULL:
            w["norm"] = _Fp8Weight(g("norm.linear.weight"), g("norm.linear.bias"), g("norm.linear_input_scale"), dev, self.dtype)
        else:
            w["norm_w"] = g("norm.linear.weight").to(device=dev, dtype=self.dtype).contiguous()
            w["norm_b"] = g("norm.linear.bias").to(device=dev, dtype=self.dtype).contiguous()
        w["qk_scale"] = torch.cat([g("attn.norm_q.weight").reshape(-1), g("attn.norm_k.weight").reshape(-1)]).to(
            device=dev, dtype=self.dtype).contiguous()
        if w["qkv"].n != 3 * self.dim or w["mlp"].n != self.mlp_scale * self.dim or w["out"].k != (self.mlp_scale + 1) * self.dim:
            raise RuntimeError("weight shapes do not match the block's dimensions")
        self._w = w

    def _buffer(self, name, shape, dtype, device):
        t = self._buf.get(name)
        if t is None or tuple(t.shape) != tuple(shape) or t.dtype != dtype or t.device != device:
            t = torch.empty(shape, dtype=dtype, device=device)
            self._buf[name] = t
        return t

    def forward(self, hidden_states, rope_emb, temb):
        """hidden_states [B, S, D], rope_emb [B, S, head_dim/2, 2, 2] (any shape with that many elements), temb [B, D]
        already SiLU'd; all CUDA, contiguous and of the inference dtype (FluxSingleTransformerBlockOp.cc:40-62).
        Returns a new [B, S, D] tensor owned by torch."""
        if self._w is None:
            raise RuntimeError("weights not loaded")
        for t in (hidden_states, rope_emb, temb):
            if not (t.is_cuda and t.is_contiguous() and t.dtype == self.dtype):
                raise RuntimeError("inputs must be contiguous CUDA tensors of the inference dtype")
        B, S, D = hidden_states.shape
        if D != self.dim or tuple(temb.shape) != (B, D) or rope_emb.numel() != B * S * self.head_dim * 2:
            raise RuntimeError("shape mismatch")
        w, dev, dt = self._w, hidden_states.device, self.dtype
        T = B * S

        # ---- modulation: msa = linear(temb) -> shift | scale | gate
        if self.quant_level == FP8_W8A8_FULL:
            nw = w["norm"]
            tq = self._buffer("temb_q", (B, D), torch.uint8, dev)
            ops.invoke_cuda_d2d_scale_cpy_convert(tq, temb, nw.input_scale)
            msa = self._buffer("msa", (B, 3 * D), dt, dev)
            ops.gemm_with_residual_and_bias_fp8(nw.qweight, nw.w_scale, tq, nw.input_scale, msa, bias=nw.bias)
        else:
            msa = torch.addmm(w["norm_b"], temb, w["norm_w"].t())
        shift, scale, gate = (c.contiguous() for c in msa.chunk(3, dim=1))

        # ---- AdaLN modulation, 16-bit result and its e4m3 form for to_qkv in one pass
        norm = self._buffer("norm", (B, S, D), dt, dev)
        norm_q = self._buffer("norm_q", (T, D), torch.uint8, dev)
        ops.invoke_layer_norm_with_shift_and_scale(norm, hidden_states, scale, shift, eps=1e-6, qf8=norm_q,
                                                   f8_scale=w["qkv"].input_scale)

        # ---- attention branch
        qkv = self._buffer("qkv", (T, 3 * D), dt, dev)
        ops.gemm_with_residual_and_bias_fp8(w["qkv"].qweight, w["qkv"].w_scale, norm_q, w["qkv"].input_scale, qkv, bias=w["qkv"].bias)
        ops.invoke_fused_rmsnorm_and_rope(qkv, qkv, w["qk_scale"], rope_emb, 1e-6, B, S, self.heads, self.head_dim)
        v5 = qkv.view(B, S, 3, self.heads, self.head_dim)
        q, k, v = (v5[:, :, i].transpose(1, 2) for i in range(3))          # [B, H, S, Dh] views of the packed buffer
        attn = torch.nn.functional.scaled_dot_product_attention(q, k, v)    # library attention (outside this path)
        attn = attn.transpose(1, 2).reshape(T, D)

        # ---- proj_out input [T, (mlp_scale + 1) * D] in e4m3, filled in place by its two producers
        cat8 = self._buffer("cat8", (T, (self.mlp_scale + 1) * D), torch.uint8, dev)
        ops.quant_fp8_into_columns(cat8, 0, attn, w["out"].input_scale)
        mlp_in = self._buffer("mlp_in", (T, D), torch.uint8, dev)
        ops.invoke_cuda_d2d_scale_cpy_convert(mlp_in, norm.view(T, D), w["mlp"].input_scale)
        ops.gemm_fp8_quant_into_columns(w["mlp"].qweight, w["mlp"].w_scale, mlp_in, w["mlp"].input_scale, cat8, D,
                                        w["out"].input_scale, dt, bias=w["mlp"].bias, is_gelu=True)

        # ---- proj_out, then gate and residual
        y = self._buffer("y", (T, D), dt, dev)
        ops.gemm_with_residual_and_bias_fp8(w["out"].qweight, w["out"].w_scale, cat8, w["out"].input_scale, y, bias=w["out"].bias)
        out = torch.empty_like(hidden_states)
        ops.invoke_fused_gate_and_residual(out, y.view(B, S, D), gate, hidden_states)
        return out

    __call__ = forward
