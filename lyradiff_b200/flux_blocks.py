"""Python mirrors of the reference's block-level torch custom classes for the FLUX blocks.

FluxTransformerBlockOp (double-stream, at the end of this file) follows the same conventions as the single-stream
class described here.

`torch.classes.lyradiff.FluxSingleTransformerBlockOp` (src/lyradiff/th_op/pybind.cc:82-96,
th_op/flux_single_transformer_block/FluxSingleTransformerBlockOp.h:287-315) with the same constructor arguments,
method names and tensor conventions, running the FP8 data flow of FluxSingleTransformerFP8Block<T>::forward
(src/lyradiff/layers/flux_single_transformer_block/FluxSingleTransformerFP8Block.cc:162-310) on liblyraq.so:

    msa = linear(temb)                       -> shift, scale, gate            (temb arrives SiLU'd, AdaFP8LayerNorm.cc:100)
    norm = LN(x) * (1 + scale) + shift       -> two e4m3 forms in one kernel  (lyraq_adaln_quant_fp8x2)
    qkv = FP8 GEMM(norm_q8, to_qkv) + bias   -> QK RMSNorm + RoPE in place    (lyraq_gemm_fp8, lyraq_rmsnorm_rope)
    cat8[:, :D]  = e4m3(attention(q, k, v))                                   (lyraq_attention: tcgen05 attention forward
                                                                              with the e4m3 quantize in its epilogue)
    cat8[:, D:]  = e4m3(gelu(FP8 GEMM(e4m3(norm), proj_mlp) + bias))          (lyraq_gemm_fp8_quant_ld)
    out = gate * (FP8 GEMM(cat8, proj_out) + bias) + x                        (lyraq_gemm_fp8_gate: one launch)

The 16-bit concat buffer and its quantize pass (invokeFusedCatAndGelu + invokeCudaD2DScaleCpyConvert) do not exist here.
quant_level 1 (FP8_W8A8) keeps the modulation linear in 16 bits (a torch matmul, as the reference calls cuBLAS for it),
quant_level 2 (FP8_W8A8_FULL) runs it in FP8 too.

quant_level 7 (INT4_W4A4) and 8 (INT4_W4A4_FULL, FP8 modulation linear) of the single-stream block run the W4A4 data flow of
FluxSingleTransformerInt4Block<T>::forward (layers/flux_single_transformer_block/FluxSingleTransformerInt4Block.cc:198-322)
and FluxSingleAttentionInt4Processor<T>::forward (layers/flux_single_attention_processor/FluxSingleAttentionInt4Processor.cc:
138-192), each linear one lyraq_w4a4_lora_forward (int4 quantize + LoRA-down, then grouped GEMM + LoRA-up + epilogue):

    norm = LN(x) * (1 + scale) + shift                     16-bit                          (lyraq_adaln_quant, y only)
    qkv  = T(T(W4A4(norm, to_qkv)) + bias)                 -> QK RMSNorm + RoPE in place   (the bias add of
                                                                                           fuseBiasRmsNormAndRope)
    mlp  = T(gelu(T(T(W4A4(norm, proj_mlp)) + bias)))                                      (invokeFusedBiasAndGelu)
    h    = T(T(W4A4(mlp, proj_out.linears.1.linear)) + T(T(W4A4(attn, proj_out.linears.0)) + bias))
                                                                                           (invokeFusedBiasAndResidual)
    out  = T(T(h * gate) + x)                                                              (lyraq_gate_residual)

with the roundings of the reference's separate 16-bit kernels kept inside the GEMM epilogues (LYRAQ_EPI_ROUND_EACH).
Other quant levels are not built: the constructors raise NotImplementedError.  LoRA hot-swap (load_lora_by_name,
clear_lora) re-merges from a host copy of the 16-bit weight and re-quantizes, as the reference's FP8 layers do;
reload_model_from_bin reads the reference's raw .bin files.
"""

import os
import warnings

import numpy as np
import torch

from . import layers, ops

_DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16}
FP8_W8A8, FP8_W8A8_FULL, INT4_W4A4, INT4_W4A4_FULL = 1, 2, 7, 8


class LyraDiffCommonContext:
    """LyraDiffCommonContext (src/lyradiff/th_op/lyradiff_common_context/LyraDiffCommonContext.h:23-38): the reference's
    owner of stream, allocator and cuBLAS handles.  Here the kernels run on torch's current stream and buffers are torch
    tensors, so the context carries nothing."""

    def __init__(self):
        pass


class _Fp8Weight:
    """One quantized linear as MACROLoadFP8WeightFromCache leaves it (src/lyradiff/utils/common_macro_def.h:76-92): e4m3
    weight with its amax / 448 scale, bias, static input scale, and a host copy of the 16-bit weight that every LoRA merge
    starts from (FP8LoraWeight<T>, src/lyradiff/interface/IFLoraWeight.h:81-133)."""

    def __init__(self, weight, bias, input_scale, device, dtype):
        w = weight.to(device=device, dtype=dtype).contiguous()
        self.n, self.k = w.shape
        self.weight_h = w.to("cpu")
        self.qweight = torch.empty(self.n, self.k, dtype=torch.uint8, device=device)
        self.w_scale = torch.empty(1, dtype=torch.float32, device=device)
        ops.weight_quant_fp8(self.qweight, self.w_scale, w)
        self.bias = None if bias is None else bias.to(device=device, dtype=dtype).contiguous()
        self.input_scale = input_scale.to(device=device, dtype=torch.float32).reshape(1).contiguous()
        self.loaded_lora = False

    def load_lora(self, lora_weight, scale):
        """weight_h + lora * scale (16-bit arithmetic), then a fresh amax scale and e4m3 cast; merges do not stack."""
        w = self.weight_h.to(self.qweight.device)
        ops.invoke_load_lora(w, lora_weight.to(device=w.device, dtype=w.dtype).reshape(w.shape).contiguous(), scale)
        ops.weight_quant_fp8(self.qweight, self.w_scale, w)
        self.loaded_lora = True

    def clear_lora(self):
        if self.loaded_lora:
            ops.weight_quant_fp8(self.qweight, self.w_scale, self.weight_h.to(self.qweight.device))
            self.loaded_lora = False


class _Linear16:
    """The 16-bit modulation linear of quant_level 1 / 7 with its host copy (LoraWeightV2<T>, IFLoraWeight.h:40-78)."""

    def __init__(self, weight, bias, device, dtype):
        self.w = weight.to(device=device, dtype=dtype).contiguous()
        self.b = bias.to(device=device, dtype=dtype).contiguous()
        self.weight_h = self.w.to("cpu")
        self.loaded_lora = False

    def load_lora(self, lora_weight, scale):
        self.w.copy_(self.weight_h)
        ops.invoke_load_lora(self.w, lora_weight.to(device=self.w.device, dtype=self.w.dtype).reshape(self.w.shape).contiguous(), scale)
        self.loaded_lora = True

    def clear_lora(self):
        if self.loaded_lora:
            self.w.copy_(self.weight_h)
            self.loaded_lora = False


def _target_device(device):
    """`device` of reload_model_from_state_dict says where the state-dict tensors LIVE ("cpu" or "cuda...": the reference
    picks the memcpy kind from it, FluxSingleTransformerBlockOp.h:261-264, and its Python wrappers pass "cpu"); the weights
    always go to the current CUDA device.  torch knows where each tensor is, so the argument is only validated."""
    device = str(device)  # a torch.device is accepted too
    if not (device == "cpu" or device.startswith("cuda")):
        raise RuntimeError("device must be 'cpu' or 'cuda[:n]' (where the state dict's tensors are)")
    return torch.device("cuda", torch.cuda.current_device())


def _load_lora_by_name(table, names, weight, scale):
    """IFLoraWeight<T>::loadLoraByName (IFLoraWeight.h:150-173): walk the nested name table; a name that leads nowhere is
    reported and skipped, as the reference does."""
    node = table
    for name in names:
        if isinstance(node, dict) and name in node:
            node = node[name]
        else:
            warnings.warn("lora name cannot find weights to load: %s" % " ".join(names))
            return
    if isinstance(node, dict):
        warnings.warn("lora name cannot find weights to load: %s" % " ".join(names))
        return
    node.load_lora(weight, scale)


def _clear_lora(table):
    for node in table.values():
        if isinstance(node, dict):
            _clear_lora(node)
        else:
            node.clear_lora()


_BIN_DTYPES = {"fp32": np.float32, "fp16": np.float16}


def _read_bin(path, key, shape, kind, file_dtype):
    """One raw array of loadWeightFromBin (src/lyradiff/utils/memory_utils.cu:295-364): file `<path><key>.bin`, elements of
    the model file type for 16-bit tensors ("T"), fp32 for scales ("f32"), int8 for packed int4 weights ("i8").  A missing
    or short file raises (the reference logs a warning and leaves the weight uninitialised)."""
    fn = path + key + ".bin"
    dt = {"T": file_dtype, "f32": np.float32, "i8": np.int8}[kind]
    count = int(np.prod(shape))
    if not os.path.exists(fn) or os.path.getsize(fn) < count * np.dtype(dt).itemsize:
        raise RuntimeError("weight file missing or too small: %s" % fn)
    return torch.from_numpy(np.fromfile(fn, dtype=dt, count=count).reshape(shape))


def _state_dict_from_bin(path, model_dtype, manifest):
    if model_dtype not in _BIN_DTYPES:
        raise ValueError("wrong model_dtype")  # std::invalid_argument in the reference (FluxSingleTransformerBlockOp.h:241-243)
    return {key: _read_bin(path, key, shape, kind, _BIN_DTYPES[model_dtype]) for key, shape, kind in manifest}


def _fp8_linear_files(name, n, k):
    return [(name + ".weight", (n, k), "T"), (name + ".bias", (n,), "T"), (name + "_input_scale", (1,), "f32")]


def _w4a4_linear_files(name, n, k, has_bias=True):
    files = [(name + "packed_weight", (n, k // 2), "i8"), (name + "weight_scale", (n, k // 64), "f32"),
             (name + "lora_up", (n, 32), "T"), (name + "lora_down", (32, k), "T"), (name + "smooth", (k,), "f32")]
    return files + ([(name + "bias", (n,), "T")] if has_bias else [])


def _modulation_files(name, chunks, D, fp8):
    files = [(name + ".weight", (chunks * D, D), "T"), (name + ".bias", (chunks * D,), "T")]
    return files + ([(name + "_input_scale", (1,), "f32")] if fp8 else [])


def _w4a4_from_state_dict(sd, name, n, k, device, dtype, has_bias, gelu=False):
    """One W4A4 linear from the tensors W4A4GemmWeight<T>::loadWeights reads (src/lyradiff/layers/w4a4_gemm_block/
    W4A4GemmWeight.cc:62-79; the reference's own state-dict loader for this layer is empty, so the .bin names serve as
    keys): `<name>packed_weight` int8/uint8 [n, k/2], `<name>weight_scale` fp32 (or fp16) [n, k/64], `<name>smooth`
    fp32 [k], `<name>lora_down` [32, k], `<name>lora_up` [n, 32], `<name>bias` [n] where the layer has one."""
    pw = sd[name + "packed_weight"].to(device).contiguous().view(torch.uint8).reshape(n, k // 2)
    ws = sd[name + "weight_scale"].to(device).contiguous().reshape(n, k // 64)
    if ws.dtype not in (torch.float32, torch.float16):
        ws = ws.float()
    smooth = sd[name + "smooth"].to(device=device, dtype=torch.float32).contiguous()
    down = sd[name + "lora_down"].to(device=device, dtype=dtype).contiguous().reshape(32, k)
    up = sd[name + "lora_up"].to(device=device, dtype=dtype).contiguous().reshape(n, 32)
    bias = sd[name + "bias"].to(device=device, dtype=dtype).contiguous() if has_bias else None
    return layers.W4A4Gemm(pw, ws, smooth, bias, gelu=gelu, lora_down=down, lora_up=up, round_each=True)


class FluxSingleTransformerBlockOp:
    def __init__(self, inference_dtype="bf16", embedding_dim=3072, embedding_head_num=24, embedding_head_dim=128, mlp_scale=4,
                 quant_level=0):
        if inference_dtype not in _DTYPES:
            raise RuntimeError("inference_dtype must be 'bf16' or 'fp16'")
        if quant_level not in (FP8_W8A8, FP8_W8A8_FULL, INT4_W4A4, INT4_W4A4_FULL):
            raise NotImplementedError("quant_level %r: only 1, 2 (FP8) and 7, 8 (INT4 W4A4) are built here; the 16-bit level 0 (the "
                                      "reference's default) and FP8 weight-only level 3 stay with the reference's own library" % (quant_level,))
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
        """FluxSingleTransformer*BlockWeight<T>::loadWeights: one raw file `<path><key>.bin` per tensor, keys as in
        reload_model_from_state_dict, 16-bit tensors stored as `dtype` ("fp32" or "fp16"), scales as fp32, packed int4
        weights as int8 (FluxSingleTransformerFP8BlockWeight.cc:97-121, FluxSingleTransformerInt4BlockWeight.cc:70-84).
        `path` is a prefix, e.g. ".../single_transformer_blocks.0."; the weights go to the current CUDA device."""
        self.reload_model_from_state_dict("", _state_dict_from_bin(path, dtype, self._bin_files()), "cuda")

    def _bin_files(self):
        D, m = self.dim, self.mlp_scale
        full = self.quant_level in (FP8_W8A8_FULL, INT4_W4A4_FULL)
        files = _modulation_files("norm.linear", 3, D, full)
        files += [("attn.norm_q.weight", (self.head_dim,), "T"), ("attn.norm_k.weight", (self.head_dim,), "T")]
        if self.quant_level in (INT4_W4A4, INT4_W4A4_FULL):
            files += _w4a4_linear_files("attn.to_qkv.", 3 * D, D) + _w4a4_linear_files("proj_mlp.", m * D, D)
            files += _w4a4_linear_files("proj_out.linears.0.", D, D)
            files += _w4a4_linear_files("proj_out.linears.1.linear.", D, m * D, has_bias=False)
        else:
            files += _fp8_linear_files("attn.to_qkv", 3 * D, D) + _fp8_linear_files("proj_mlp", m * D, D)
            files += _fp8_linear_files("proj_out", D, (m + 1) * D)
        return files

    def _lora_table(self):
        """Names as the reference's lora_layer_map / lora_weight_map nest them (FluxSingleTransformerFP8BlockWeight.cc:33,80-89,
        FluxSingleAttentionFP8ProcessorWeight.cc:51-54, AdaFP8LayerNormWeight.cc:47-51).  The W4A4 linears have no
        hot-swap in the reference either (they carry their LoRA branch as weights)."""
        if self._w is None:
            raise RuntimeError("weights not loaded")
        w = self._w
        table = {"norm": {"linear": w["norm"] if "norm" in w else w["norm16"]}}
        if not w.get("int4"):
            table.update({"attn": {"to_qkv": w["qkv"]}, "proj_mlp": w["mlp"], "proj_out": w["out"]})
        return table

    def load_lora_by_name(self, names, weight, scale):
        """names: the path to one linear, e.g. ["attn", "to_qkv"] or ["proj_mlp"]; weight: the merged low-rank update
        (up @ down) in the layer's [n, k] layout and the inference dtype; scale: its strength."""
        _load_lora_by_name(self._lora_table(), list(names), weight, float(scale))

    def clear_lora(self):
        _clear_lora(self._lora_table())

    def reload_model_from_state_dict(self, prefix, state_dict, device):
        """Keys as the reference reads them (FluxSingleTransformerFP8BlockWeight.cc:135-149,
        FluxSingleAttentionFP8ProcessorWeight.cc:111-114): `<prefix>norm.linear.{weight,bias}`,
        `<prefix>attn.to_qkv.{weight,bias}`, `<prefix>attn.norm_q.weight`, `<prefix>attn.norm_k.weight`,
        `<prefix>proj_mlp.{weight,bias}`, `<prefix>proj_out.{weight,bias}` and the fp32 scalars
        `<prefix>attn.to_qkv_input_scale`, `<prefix>proj_mlp_input_scale`, `<prefix>proj_out_input_scale`
        (plus `<prefix>norm.linear_input_scale` at quant_level 2).  Host or device tensors; weights are quantized here."""
        dev = _target_device(device)
        sd = state_dict
        g = lambda name: sd[prefix + name]
        w = {}
        if self.quant_level in (INT4_W4A4, INT4_W4A4_FULL):
            return self._reload_int4(prefix, sd, dev)
        w["qkv"] = _Fp8Weight(g("attn.to_qkv.weight"), g("attn.to_qkv.bias"), g("attn.to_qkv_input_scale"), dev, self.dtype)
        w["mlp"] = _Fp8Weight(g("proj_mlp.weight"), g("proj_mlp.bias"), g("proj_mlp_input_scale"), dev, self.dtype)
        w["out"] = _Fp8Weight(g("proj_out.weight"), g("proj_out.bias"), g("proj_out_input_scale"), dev, self.dtype)
        if self.quant_level == FP8_W8A8_FULL:
            w["norm"] = _Fp8Weight(g("norm.linear.weight"), g("norm.linear.bias"), g("norm.linear_input_scale"), dev, self.dtype)
        else:
            w["norm16"] = _Linear16(g("norm.linear.weight"), g("norm.linear.bias"), dev, self.dtype)
        w["qk_scale"] = torch.cat([g("attn.norm_q.weight").reshape(-1), g("attn.norm_k.weight").reshape(-1)]).to(
            device=dev, dtype=self.dtype).contiguous()
        if w["qkv"].n != 3 * self.dim or w["mlp"].n != self.mlp_scale * self.dim or w["out"].k != (self.mlp_scale + 1) * self.dim:
            raise RuntimeError("weight shapes do not match the block's dimensions")
        self._w = w

    def _reload_int4(self, prefix, sd, dev):
        """Keys (FluxSingleTransformerInt4BlockWeight.cc:79-83, FluxSingleAttentionInt4ProcessorWeight.cc:73-78):
        `<prefix>norm.linear.{weight,bias}` (+ `norm.linear_input_scale` at level 8), `<prefix>attn.norm_q.weight`,
        `<prefix>attn.norm_k.weight` and the W4A4 linears `<prefix>attn.to_qkv.`, `<prefix>proj_mlp.`,
        `<prefix>proj_out.linears.0.` (all with bias) and `<prefix>proj_out.linears.1.linear.` (no bias)."""
        D, dt = self.dim, self.dtype
        g = lambda name: sd[prefix + name]
        w = {"int4": True}
        w["qkv"] = _w4a4_from_state_dict(sd, prefix + "attn.to_qkv.", 3 * D, D, dev, dt, True)
        w["mlp"] = _w4a4_from_state_dict(sd, prefix + "proj_mlp.", self.mlp_scale * D, D, dev, dt, True, gelu=True)
        w["out1"] = _w4a4_from_state_dict(sd, prefix + "proj_out.linears.0.", D, D, dev, dt, True)
        w["out2"] = _w4a4_from_state_dict(sd, prefix + "proj_out.linears.1.linear.", D, self.mlp_scale * D, dev, dt, False)
        if self.quant_level == INT4_W4A4_FULL:
            w["norm"] = _Fp8Weight(g("norm.linear.weight"), g("norm.linear.bias"), g("norm.linear_input_scale"), dev, dt)
        else:
            w["norm16"] = _Linear16(g("norm.linear.weight"), g("norm.linear.bias"), dev, dt)
        w["qk_scale"] = torch.cat([g("attn.norm_q.weight").reshape(-1), g("attn.norm_k.weight").reshape(-1)]).to(
            device=dev, dtype=dt).contiguous()
        self._w = w

    def _forward_int4(self, hidden_states, rope_emb, shift, scale, gate):
        B, S, D = hidden_states.shape
        w, dev, dt, T = self._w, hidden_states.device, self.dtype, B * S
        norm = self._buffer("norm16", (T, D), dt, dev)
        ops.invoke_layer_norm_with_shift_and_scale(norm.view(B, S, D), hidden_states, scale, shift, eps=1e-6)
        qkv = self._buffer("qkv", (T, 3 * D), dt, dev)
        w["qkv"].forward(norm, out=qkv)
        ops.invoke_fused_rmsnorm_and_rope(qkv, qkv, w["qk_scale"], rope_emb, 1e-6, B, S, self.heads, self.head_dim)
        attn = self._buffer("attn16", (T, D), dt, dev)
        ops.flash_attention(qkv, B, S, self.heads, self.head_dim, out=attn)
        mlp = self._buffer("mlp16", (T, self.mlp_scale * D), dt, dev)
        w["mlp"].forward(norm, out=mlp)
        h1 = self._buffer("h1", (T, D), dt, dev)
        w["out1"].forward(attn, out=h1)
        h = self._buffer("h", (T, D), dt, dev)
        w["out2"].forward(mlp, residual=h1, out=h)
        out = torch.empty_like(hidden_states)
        ops.invoke_fused_gate_and_residual(out, h.view(B, S, D), gate, hidden_states)
        return out

    def _buffer(self, name, shape, dtype, device):
        t = self._buf.get(name)
        if t is None or tuple(t.shape) != tuple(shape) or t.dtype != dtype or t.device != device:
            t = torch.empty(shape, dtype=dtype, device=device)
            self._buf[name] = t
        return t

    def modulation(self, temb):
        """msa = norm.linear(temb) -> [shift, scale, gate], each [B, D] contiguous.  It depends on temb alone, so a caller that
        runs many blocks with one temb (flux_model) may compute it ahead of the block, on another stream."""
        w, dev, dt = self._w, temb.device, self.dtype
        B, D = temb.shape
        if self.quant_level in (FP8_W8A8_FULL, INT4_W4A4_FULL):
            nw = w["norm"]
            tq = torch.empty(B, D, dtype=torch.uint8, device=dev)
            ops.invoke_cuda_d2d_scale_cpy_convert(tq, temb, nw.input_scale)
            msa = torch.empty(B, 3 * D, dtype=dt, device=dev)
            ops.gemm_with_residual_and_bias_fp8(nw.qweight, nw.w_scale, tq, nw.input_scale, msa, bias=nw.bias)
        else:
            msa = torch.addmm(w["norm16"].b, temb, w["norm16"].w.t())
        return [c.contiguous() for c in msa.chunk(3, dim=1)]

    def forward(self, hidden_states, rope_emb, temb, mod=None):
        """hidden_states [B, S, D], rope_emb [B, S, head_dim/2, 2, 2] (any shape with that many elements), temb [B, D]
        already SiLU'd; all CUDA, contiguous and of the inference dtype (FluxSingleTransformerBlockOp.cc:40-62).
        Returns a new [B, S, D] tensor owned by torch.  `mod` (not in the reference's signature) is an optional
        (tensors, event) pair from modulation() computed ahead on another stream."""
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
        shift, scale, gate = _take_modulation(mod) if mod is not None else self.modulation(temb)
        if w.get("int4"):
            return self._forward_int4(hidden_states, rope_emb, shift, scale, gate)

        # ---- AdaLN modulation straight into the e4m3 inputs of to_qkv and proj_mlp (their input scales differ); the
        # 16-bit result is never written
        norm_q = self._buffer("norm_q", (T, D), torch.uint8, dev)
        mlp_in = self._buffer("mlp_in", (T, D), torch.uint8, dev)
        ops.adaln_quant_fp8x2(None, norm_q, w["qkv"].input_scale, mlp_in, w["mlp"].input_scale, hidden_states, scale, shift,
                              eps=1e-6)

        # ---- attention branch
        qkv = self._buffer("qkv", (T, 3 * D), dt, dev)
        ops.gemm_with_residual_and_bias_fp8(w["qkv"].qweight, w["qkv"].w_scale, norm_q, w["qkv"].input_scale, qkv, bias=w["qkv"].bias)
        ops.invoke_fused_rmsnorm_and_rope(qkv, qkv, w["qk_scale"], rope_emb, 1e-6, B, S, self.heads, self.head_dim)

        # ---- proj_out input [T, (mlp_scale + 1) * D] in e4m3, filled in place by its two producers: the attention kernel
        # writes its output as e4m3 into the first D columns, the proj_mlp GEMM its GELU output into the rest
        cat8 = self._buffer("cat8", (T, (self.mlp_scale + 1) * D), torch.uint8, dev)
        ops.flash_attention(qkv, B, S, self.heads, self.head_dim, out=cat8, out_scale=w["out"].input_scale)
        ops.gemm_fp8_quant_into_columns(w["mlp"].qweight, w["mlp"].w_scale, mlp_in, w["mlp"].input_scale, cat8, D,
                                        w["out"].input_scale, dt, bias=w["mlp"].bias, is_gelu=True)

        # ---- proj_out with gate and residual in its epilogue (a separate kernel only where a tile would straddle batches)
        out = torch.empty_like(hidden_states)
        if not ops.gemm_fp8_gate_residual(w["out"].qweight, w["out"].w_scale, cat8, w["out"].input_scale, out.view(T, D), gate,
                                          hidden_states.view(T, D), S, bias=w["out"].bias):
            y = self._buffer("y", (T, D), dt, dev)
            ops.gemm_with_residual_and_bias_fp8(w["out"].qweight, w["out"].w_scale, cat8, w["out"].input_scale, y, bias=w["out"].bias)
            ops.invoke_fused_gate_and_residual(out, y.view(B, S, D), gate, hidden_states)
        return out

    __call__ = forward


def _take_modulation(mod):
    """A modulation computed on another stream: wait for its event on the current stream and tell the allocator that the
    tensors are used here too."""
    tensors, event = mod
    cur = torch.cuda.current_stream()
    cur.wait_event(event)
    for t in tensors:
        t.record_stream(cur)
    return tensors


def _modulation(op, w, temb, chunks):
    """msa = linear(temb) -> `chunks` contiguous [B, D] tensors (AdaFP8LayerNorm<T>::forward,
    src/lyradiff/layers/ada_layer_norm/AdaFP8LayerNorm.cc:96-160)."""
    B, D = temb.shape
    if "fp8" in w:
        nw = w["fp8"]
        tq = torch.empty(B, D, dtype=torch.uint8, device=temb.device)
        ops.invoke_cuda_d2d_scale_cpy_convert(tq, temb, nw.input_scale)
        msa = torch.empty(B, chunks * D, dtype=op.dtype, device=temb.device)
        ops.gemm_with_residual_and_bias_fp8(nw.qweight, nw.w_scale, tq, nw.input_scale, msa, bias=nw.bias)
    else:
        msa = torch.addmm(w["lin16"].b, temb, w["lin16"].w.t())
    return [c.contiguous() for c in msa.chunk(chunks, dim=1)]


class FluxTransformerBlockOp:
    """torch.classes.lyradiff.FluxTransformerBlockOp (src/lyradiff/th_op/pybind.cc:66-80,
    th_op/flux_transformer_block/FluxTransformerBlockOp.h:187-237): the double-stream block.  Data flow of
    FluxTransformerFP8Block<T>::forward (src/lyradiff/layers/flux_transformer_block/FluxTransformerFP8Block.cc:155-245),
    FluxAttentionFP8Processor<T>::forward (layers/flux_attention_processor/FluxAttentionFP8Processor.cc:140-340) and
    FluxAttnPostFP8Processor<T>::forward (layers/flux_attn_post_processor/FluxAttnPostFP8Processor.cc:90-205), per stream
    (image tokens `hidden`, text tokens `encoder`):

        shift, scale, gate, shift2, scale2, gate2 = linear(temb)
        qkv  = FP8 GEMM(e4m3(LN(x)(1+scale)+shift), to_qkv) + bias        (AdaLN + quantize in one kernel)
        both streams: QK RMSNorm + RoPE into one [B, S_txt + S_img] buffer (text first), joint attention (lyraq_attention, e4m3 out per stream)
        h    = x + gate * (FP8 GEMM(e4m3(attn), to_out) + bias)
        ff   = FP8 GEMM(e4m3(gelu(FP8 GEMM(e4m3(LN(h)(1+scale2)+shift2), net.0.proj) + bias)), net.2) + bias
        out  = h + gate2 * ff              (the quantize between the two FF linears is fused into the first GEMM's epilogue)

    quant_level 7 / 8 (FluxTransformerInt4Block.cc:155-240, FluxAttentionInt4Processor.cc:157-305,
    FluxAttnPostInt4Processor.cc forward): to_qkv, to_out and net.0.proj of each stream are W4A4 linears with LoRA (their
    bias added by a 16-bit kernel in the reference, kept as a rounding step here), AdaLN outputs stay 16-bit, and net.2
    stays an FP8 linear fed by an e4m3 quantize of the GELU output.
    """

    def __init__(self, inference_dtype="bf16", embedding_dim=3072, embedding_head_num=24, embedding_head_dim=128, mlp_scale=6,
                 quant_level=0):
        if inference_dtype not in _DTYPES:
            raise RuntimeError("inference_dtype must be 'bf16' or 'fp16'")
        if quant_level not in (FP8_W8A8, FP8_W8A8_FULL, INT4_W4A4, INT4_W4A4_FULL):
            raise NotImplementedError("quant_level %r: only 1, 2 (FP8) and 7, 8 (INT4 W4A4) are built here; the 16-bit level 0 (the "
                                      "reference's default) and FP8 weight-only level 3 stay with the reference's own library" % (quant_level,))
        if embedding_head_num * embedding_head_dim != embedding_dim:
            raise RuntimeError("embedding_dim must equal embedding_head_num * embedding_head_dim")
        self.dtype = _DTYPES[inference_dtype]
        self.dim, self.heads, self.head_dim, self.mlp_scale = embedding_dim, embedding_head_num, embedding_head_dim, mlp_scale
        self.quant_level = quant_level
        self._w = None

    def initialize(self, ctx):
        self._ctx = ctx

    _STREAMS = (("norm1", "attn.to_qkv", "attn.to_out.0", "attn.norm_q.weight", "attn.norm_k.weight", "ff"),
                ("norm1_context", "attn.to_added_qkv", "attn.to_add_out", "attn.norm_added_q.weight", "attn.norm_added_k.weight",
                 "ff_context"))

    def reload_model_from_bin(self, path, dtype):
        """FluxTransformer*BlockWeight<T>::loadWeights (FluxTransformerFP8BlockWeight.cc:84-100,
        FluxTransformerInt4BlockWeight.cc:78-91): `<path><key>.bin` per tensor, keys as in reload_model_from_state_dict."""
        self.reload_model_from_state_dict("", _state_dict_from_bin(path, dtype, self._bin_files()), "cuda")

    def _bin_files(self):
        D = self.dim
        int4 = self.quant_level in (INT4_W4A4, INT4_W4A4_FULL)
        files = []
        for norm, qkv, out, nq, nk, ff in self._STREAMS:
            files += _modulation_files(norm + ".linear", 6, D, self.quant_level in (FP8_W8A8_FULL, INT4_W4A4_FULL))
            files += [(nq, (self.head_dim,), "T"), (nk, (self.head_dim,), "T")]
            if int4:
                files += _w4a4_linear_files(qkv + ".", 3 * D, D) + _w4a4_linear_files(out + ".", D, D)
                files += _w4a4_linear_files(ff + ".net.0.proj.", 4 * D, D)
            else:
                files += _fp8_linear_files(qkv, 3 * D, D) + _fp8_linear_files(out, D, D) + _fp8_linear_files(ff + ".net.0.proj", 4 * D, D)
            files += _fp8_linear_files(ff + ".net.2", D, 4 * D)
        return files

    def _lora_table(self):
        """FluxTransformerFP8BlockWeight.cc:41-45, FluxAttentionFP8ProcessorWeight.cc:91-108,
        FluxAttnPostFP8ProcessorWeight.cc:58-64, AdaFP8LayerNormWeight.cc:47-51."""
        if self._w is None:
            raise RuntimeError("weights not loaded")
        wi, wt = self._w["img"], self._w["txt"]
        mod = lambda w: {"linear": w["norm"].get("fp8") or w["norm"]["lin16"]}
        table = {"norm1": mod(wi), "norm1_context": mod(wt), "ff": {"net.2": wi["ff2"]}, "ff_context": {"net.2": wt["ff2"]}}
        if not wi.get("int4"):
            table["attn"] = {"to_qkv": wi["qkv"], "to_out.0": wi["out"], "to_added_qkv": wt["qkv"], "to_add_out": wt["out"]}
            table["ff"]["net.0.proj"] = wi["ff1"]
            table["ff_context"]["net.0.proj"] = wt["ff1"]
        return table

    def load_lora_by_name(self, names, weight, scale):
        _load_lora_by_name(self._lora_table(), list(names), weight, float(scale))

    def clear_lora(self):
        _clear_lora(self._lora_table())

    def reload_model_from_state_dict(self, prefix, state_dict, device):
        """Keys (FluxTransformerFP8BlockWeight.cc:104-108 and the loaders it calls): per stream
        `norm1[_context].linear`, `attn.to_qkv | attn.to_added_qkv`, `attn.to_out.0 | attn.to_add_out`,
        `attn.norm_q, norm_k | attn.norm_added_q, norm_added_k`, `ff[_context].net.0.proj`, `ff[_context].net.2`; every
        quantized linear X has X.weight, X.bias and the fp32 scalar X_input_scale."""
        dev = _target_device(device)
        g = lambda name: state_dict[prefix + name]

        def lin(name):
            return _Fp8Weight(g(name + ".weight"), g(name + ".bias"), g(name + "_input_scale"), dev, self.dtype)

        int4 = self.quant_level in (INT4_W4A4, INT4_W4A4_FULL)
        D = self.dim

        def stream(norm, qkv, out, nq, nk, ff):
            if int4:
                # W4A4 linears under the .bin names of W4A4GemmWeight (FluxAttentionInt4ProcessorWeight.cc:63-66,
                # FluxAttnPostInt4ProcessorWeight.cc:94-96); net.2 as in the FP8 block
                w = {"int4": True,
                     "qkv": _w4a4_from_state_dict(state_dict, prefix + qkv + ".", 3 * D, D, dev, self.dtype, True),
                     "out": _w4a4_from_state_dict(state_dict, prefix + out + ".", D, D, dev, self.dtype, True),
                     "ff1": _w4a4_from_state_dict(state_dict, prefix + ff + ".net.0.proj.", 4 * D, D, dev, self.dtype, True, gelu=True),
                     "ff2": lin(ff + ".net.2")}
            else:
                w = {"qkv": lin(qkv), "out": lin(out), "ff1": lin(ff + ".net.0.proj"), "ff2": lin(ff + ".net.2")}
            if self.quant_level in (FP8_W8A8_FULL, INT4_W4A4_FULL):
                w["norm"] = {"fp8": lin(norm + ".linear")}
            else:
                w["norm"] = {"lin16": _Linear16(g(norm + ".linear.weight"), g(norm + ".linear.bias"), dev, self.dtype)}
            w["qk_scale"] = torch.cat([g(nq).reshape(-1), g(nk).reshape(-1)]).to(device=dev, dtype=self.dtype).contiguous()
            return w

        self._w = {
            "img": stream("norm1", "attn.to_qkv", "attn.to_out.0", "attn.norm_q.weight", "attn.norm_k.weight", "ff"),
            "txt": stream("norm1_context", "attn.to_added_qkv", "attn.to_add_out", "attn.norm_added_q.weight",
                          "attn.norm_added_k.weight", "ff_context"),
        }

    def modulation(self, temb):
        """(image-stream, text-stream) modulations, six [B, D] tensors each; see FluxSingleTransformerBlockOp.modulation."""
        return [_modulation(self, self._w[s]["norm"], temb, 6) for s in ("img", "txt")]

    def _pre_attention(self, w, x, temb, mod=None):
        B, S, D = x.shape
        mod = _modulation(self, w["norm"], temb, 6) if mod is None else mod
        if w.get("int4"):
            norm = torch.empty(B, S, D, dtype=self.dtype, device=x.device)
            ops.invoke_layer_norm_with_shift_and_scale(norm, x, mod[1], mod[0], eps=1e-6)
            return mod, w["qkv"].forward(norm.view(B * S, D))
        norm_q = torch.empty(B * S, D, dtype=torch.uint8, device=x.device)
        ops.invoke_layer_norm_with_shift_and_scale(None, x, mod[1], mod[0], eps=1e-6, qf8=norm_q, f8_scale=w["qkv"].input_scale)
        qkv = torch.empty(B * S, 3 * D, dtype=self.dtype, device=x.device)
        ops.gemm_with_residual_and_bias_fp8(w["qkv"].qweight, w["qkv"].w_scale, norm_q, w["qkv"].input_scale, qkv, bias=w["qkv"].bias)
        return mod, qkv

    def _post_attention(self, w, x, attn, mod):
        B, S, D = x.shape
        T = B * S
        dev, dt = x.device, self.dtype
        if w.get("int4"):
            return self._post_attention_int4(w, x, attn, mod)
        aq = attn                                  # e4m3 codes, quantized with to_out's input scale by the attention kernel
        y = torch.empty(T, D, dtype=dt, device=dev)
        h = torch.empty_like(x)
        if not ops.gemm_fp8_gate_residual(w["out"].qweight, w["out"].w_scale, aq, w["out"].input_scale, h.view(T, D), mod[2],
                                          x.view(T, D), S, bias=w["out"].bias):
            ops.gemm_with_residual_and_bias_fp8(w["out"].qweight, w["out"].w_scale, aq, w["out"].input_scale, y, bias=w["out"].bias)
            ops.invoke_fused_gate_and_residual(h, y.view(B, S, D), mod[2], x)
        nq = torch.empty(T, D, dtype=torch.uint8, device=dev)
        ops.invoke_layer_norm_with_shift_and_scale(None, h, mod[4], mod[3], eps=1e-6, qf8=nq, f8_scale=w["ff1"].input_scale)
        f1 = torch.empty(T, w["ff1"].n, dtype=torch.uint8, device=dev)
        ops.gemm_fp8_quant_out(w["ff1"].qweight, w["ff1"].w_scale, nq, w["ff1"].input_scale, f1, w["ff2"].input_scale, dt,
                               bias=w["ff1"].bias, is_gelu=True)
        out = torch.empty_like(x)
        if not ops.gemm_fp8_gate_residual(w["ff2"].qweight, w["ff2"].w_scale, f1, w["ff2"].input_scale, out.view(T, D), mod[5],
                                          h.view(T, D), S, bias=w["ff2"].bias):
            ops.gemm_with_residual_and_bias_fp8(w["ff2"].qweight, w["ff2"].w_scale, f1, w["ff2"].input_scale, y, bias=w["ff2"].bias)
            ops.invoke_fused_gate_and_residual(out, y.view(B, S, D), mod[5], h)
        return out

    def _post_attention_int4(self, w, x, attn, mod):
        B, S, D = x.shape
        T = B * S
        dev, dt = x.device, self.dtype
        ao = w["out"].forward(attn)                                    # T(T(acc) + bias): to_out + invokeAddBias
        h = torch.empty_like(x)
        ops.invoke_fused_gate_and_residual(h, ao.view(B, S, D), mod[2], x)
        n2 = torch.empty_like(x)
        ops.invoke_layer_norm_with_shift_and_scale(n2, h, mod[4], mod[3], eps=1e-6)
        f1 = w["ff1"].forward(n2.view(T, D))                           # T(gelu(T(T(acc) + bias))): invokeFusedBiasAndGelu
        f1q = torch.empty(T, 4 * D, dtype=torch.uint8, device=dev)
        ops.invoke_cuda_d2d_scale_cpy_convert(f1q, f1, w["ff2"].input_scale)
        out = torch.empty_like(x)
        if not ops.gemm_fp8_gate_residual(w["ff2"].qweight, w["ff2"].w_scale, f1q, w["ff2"].input_scale, out.view(T, D), mod[5],
                                          h.view(T, D), S, bias=w["ff2"].bias):
            y = torch.empty(T, D, dtype=dt, device=dev)
            ops.gemm_with_residual_and_bias_fp8(w["ff2"].qweight, w["ff2"].w_scale, f1q, w["ff2"].input_scale, y, bias=w["ff2"].bias)
            ops.invoke_fused_gate_and_residual(out, y.view(B, S, D), mod[5], h)
        return out

    def forward(self, hidden_states, encoder_hidden_states, rope_emb, temb, mod=None):
        """hidden_states [B, S_img, D], encoder_hidden_states [B, S_txt, D], rope_emb over the S_txt + S_img joint
        sequence (text first) with B * (S_txt + S_img) * head_dim * 2 elements, temb [B, D] SiLU'd.
        Returns [hidden_out, encoder_out]."""
        if self._w is None:
            raise RuntimeError("weights not loaded")
        for t in (hidden_states, encoder_hidden_states, rope_emb, temb):
            if not (t.is_cuda and t.is_contiguous() and t.dtype == self.dtype):
                raise RuntimeError("inputs must be contiguous CUDA tensors of the inference dtype")
        B, S, D = hidden_states.shape
        E = encoder_hidden_states.shape[1]
        if D != self.dim or encoder_hidden_states.shape[0] != B or encoder_hidden_states.shape[2] != D or \
                tuple(temb.shape) != (B, D) or rope_emb.numel() != B * (S + E) * self.head_dim * 2:
            raise RuntimeError("shape mismatch")
        wi, wt = self._w["img"], self._w["txt"]
        pre_i = pre_t = None
        if mod is not None:   # ((image tensors, text tensors), event) computed ahead on another stream
            (pre_i, pre_t), event = mod
            _take_modulation((list(pre_i) + list(pre_t), event))
        mod_i, qkv_i = self._pre_attention(wi, hidden_states, temb, pre_i)
        mod_t, qkv_t = self._pre_attention(wt, encoder_hidden_states, temb, pre_t)
        # joint sequence [B, E + S, 3, H, Dh], text first (invokeFusedRmsNormCatAndRope, flux_apply_rope.cu:78-156)
        tot = E + S
        joint = torch.empty(B, tot, 3 * D, dtype=self.dtype, device=hidden_states.device)
        rope = rope_emb.view(B, tot, self.head_dim * 2)
        qt, qi = qkv_t.view(B, E, 3 * D), qkv_i.view(B, S, 3 * D)
        for b in range(B):
            ops.invoke_fused_rmsnorm_and_rope(joint[b, :E], qt[b], wt["qk_scale"], rope[b, :E], 1e-6, 1, E, self.heads, self.head_dim)
            ops.invoke_fused_rmsnorm_and_rope(joint[b, E:], qi[b], wi["qk_scale"], rope[b, E:], 1e-6, 1, S, self.heads, self.head_dim)
        # one attention over the joint sequence; text rows and image rows leave as the inputs of the two to_out linears:
        # e4m3 with each linear's input scale (FP8), or 16-bit for the W4A4 linears, which quantize their own input
        int4 = bool(wi.get("int4"))
        adt = self.dtype if int4 else torch.uint8
        attn_t = torch.empty(B * E, D, dtype=adt, device=hidden_states.device)
        attn_i = torch.empty(B * S, D, dtype=adt, device=hidden_states.device)
        ops.flash_attention(joint.view(B * tot, 3 * D), B, tot, self.heads, self.head_dim, out=attn_t,
                            out_scale=None if int4 else wt["out"].input_scale, out2=attn_i,
                            out2_scale=None if int4 else wi["out"].input_scale, split=E)
        out_i = self._post_attention(wi, hidden_states, attn_i, mod_i)
        out_t = self._post_attention(wt, encoder_hidden_states, attn_t, mod_t)
        return [out_i, out_t]

    __call__ = forward
