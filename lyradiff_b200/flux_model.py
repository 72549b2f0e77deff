"""Python mirror of the reference's whole-model torch custom class `torch.classes.lyradiff.FluxTransformer2DModelOp`
(src/lyradiff/th_op/pybind.cc:13-44, th_op/flux_transformer_2d_model/FluxTransformer2DModelOp.cc:65-154): the same
constructor arguments, method names and state-dict keys, running FluxTransformer2DModel<T>::transformer_forward
(src/lyradiff/models/flux_transformer_2d_model/FluxTransformer2DModel.cc:230-515):

    temb   = silu(timestep_embedder(proj(timestep)) + guidance_embedder(proj(guidance)) + text_embedder(pooled))
    h, c   = x_embedder(hidden), context_embedder(encoder_hidden)
    h, c   = double-stream block i (h, c, rope, temb)            i < num_layers        (+ ControlNet residual on h)
    x      = cat(c, h) -> single-stream block j (x, rope, temb)  j < num_single_layers
    out    = proj_out(LN(h) * (1 + scale) + shift),  scale | shift = norm_out.linear(temb)

The quantized blocks are the ones of flux_blocks.py (liblyraq.so kernels).  What the reference runs in 16 bits through cuBLAS
-- the three small embedders, x_embedder, context_embedder, norm_out.linear and proj_out -- runs here through torch matmuls
(library code on both sides); the final AdaLN is lyraq_adaln_quant with its 16-bit output, the ControlNet residual is
lyraq_load_lora with alpha 1 (the reference calls invokeLoadLora for it, FluxTransformer2DModel.cc:389).  The reference's
current Python wrapper (lyradiff_flux_transformer_model_v2.py) does not use this class: it keeps these outer layers in
PyTorch and calls the per-block classes; this mirror is for callers of the older whole-model entry point.
"""

import math

import torch

from . import flux_blocks, ops
from .flux_blocks import (_DTYPES, FP8_W8A8, FP8_W8A8_FULL, INT4_W4A4, INT4_W4A4_FULL, _clear_lora, _Linear16, _load_lora_by_name,
                          _state_dict_from_bin)


def time_exponents(channels, device, max_period=10000.0):
    """The frequency table of TimeProjection<T> (src/lyradiff/layers/time_proj/TimeProjection.cc:39-51): expf(factor * i) with
    factor = -logf(max_period) / half, single precision on the host, kept on the device.  The C library's logf / expf are
    called directly (as the reference and the C++ class do): a vectorised exp may differ from them in the last bit, which at
    guidance values in the thousands moves a rounding of the projection and, through temb, every block's modulation."""
    import ctypes
    import ctypes.util
    libm = ctypes.CDLL(ctypes.util.find_library("m") or "libm.so.6")
    for f in (libm.expf, libm.logf):
        f.restype, f.argtypes = ctypes.c_float, [ctypes.c_float]
    half = channels // 2
    factor = ctypes.c_float(-libm.logf(ctypes.c_float(max_period)) / half).value
    table = [libm.expf(ctypes.c_float(ctypes.c_float(factor * i).value)) for i in range(half)]
    return torch.tensor(table, dtype=torch.float32).to(device)


def time_projection(value, exponents, dtype):
    """TimeProjection<T>(channels, flip_sin_to_cos=true, downscale_freq_shift=0) (kernel kernels/time_proj/
    time_proj_kernels.cu:70-97): sin / cos of exponent * value in fp32, cast to T, the cosine half first.  Device work only
    (no host-to-device copy), so a forward can be captured into a CUDA graph."""
    arg = exponents * float(value)
    return torch.cat([torch.cos(arg), torch.sin(arg)]).to(dtype).reshape(1, 2 * exponents.numel())


class _Mlp16:
    """TimestepEmbeddingBlock<T> (src/lyradiff/layers/timestep_embedding_block/TimestepEmbeddingBlock.cc forward):
    linear_1 -> T(h + bias) -> SiLU -> linear_2 + bias, all in 16 bits."""

    def __init__(self, sd, prefix, device, dtype):
        self.l1 = _Linear16(sd[prefix + "linear_1.weight"], sd[prefix + "linear_1.bias"], device, dtype)
        self.l2 = _Linear16(sd[prefix + "linear_2.weight"], sd[prefix + "linear_2.bias"], device, dtype)

    def __call__(self, x):
        h = torch.nn.functional.silu(torch.matmul(x, self.l1.w.t()) + self.l1.b)
        return torch.addmm(self.l2.b, h, self.l2.w.t())

    def lora_table(self):
        return {"linear_1": self.l1, "linear_2": self.l2}


def _mlp_files(prefix, d_in, d):
    return [(prefix + "linear_1.weight", (d, d_in), "T"), (prefix + "linear_1.bias", (d,), "T"),
            (prefix + "linear_2.weight", (d, d), "T"), (prefix + "linear_2.bias", (d,), "T")]


class FluxTransformer2DModelOp:
    def __init__(self, inference_dtype="bf16", input_channels=64, num_layers=19, num_single_layers=38, attention_head_dim=128,
                 num_attention_heads=24, pooled_projection_dim=768, joint_attention_dim=4096, guidance_embeds=True, quant_level=0):
        if inference_dtype not in _DTYPES:
            raise RuntimeError("inference_dtype must be 'bf16' or 'fp16'")
        if quant_level not in (FP8_W8A8, FP8_W8A8_FULL, INT4_W4A4, INT4_W4A4_FULL):
            raise NotImplementedError("quant_level %r: only 1, 2 (FP8) and 7, 8 (INT4 W4A4) are built here; the 16-bit level 0 (the "
                                      "reference's default) and FP8 weight-only level 3 stay with the reference's own library" % (quant_level,))
        if not guidance_embeds:
            raise NotImplementedError("the model is built with the guidance embedder, as the reference's C++ model is")
        self.dtype_name, self.dtype = inference_dtype, _DTYPES[inference_dtype]
        self.in_ch, self.n_double, self.n_single = input_channels, num_layers, num_single_layers
        self.head_dim, self.heads = attention_head_dim, num_attention_heads
        self.dim = attention_head_dim * num_attention_heads
        self.pooled_dim, self.joint_dim, self.quant_level = pooled_projection_dim, joint_attention_dim, quant_level
        mk = lambda cls, mlp: cls(inference_dtype, self.dim, self.heads, self.head_dim, mlp, quant_level)
        self.double_blocks = [mk(flux_blocks.FluxTransformerBlockOp, 6) for _ in range(num_layers)]
        self.single_blocks = [mk(flux_blocks.FluxSingleTransformerBlockOp, 4) for _ in range(num_single_layers)]
        self._w = None
        self._side = None
        self.overlap_modulation = True   # False: the modulation linears are issued on the caller's stream, in front of the blocks

    # ---- reference method names (th_op/pybind.cc:13-44)
    def initialize(self, ctx):
        for b in self.double_blocks + self.single_blocks:
            b.initialize(ctx)

    def reload_transformer_model_from_state_dict(self, weights, device):
        """Keys of FluxTransformer2DModelWeight<T>::loadWeightsFromCache (FluxTransformer2DModelWeight.cc:297-337):
        `x_embedder`, `context_embedder`, `proj_out` (.weight / .bias), `time_text_embed.{timestep,guidance,text}_embedder.
        linear_{1,2}`, `norm_out.linear`, `transformer_blocks.<i>.*` and `single_transformer_blocks.<j>.*` as the block classes
        read them."""
        dev, dt, sd = flux_blocks._target_device(device), self.dtype, weights
        w = {name: _Linear16(sd[name + ".weight"], sd[name + ".bias"], dev, dt) for name in ("x_embedder", "context_embedder", "proj_out")}
        for name in ("timestep_embedder", "guidance_embedder", "text_embedder"):
            w[name] = _Mlp16(sd, "time_text_embed." + name + ".", dev, dt)
        w["norm_out"] = _Linear16(sd["norm_out.linear.weight"], sd["norm_out.linear.bias"], dev, dt)
        w["exponents"] = time_exponents(256, dev)
        for i, b in enumerate(self.double_blocks):
            b.reload_model_from_state_dict("transformer_blocks.%d." % i, sd, device)
        for j, b in enumerate(self.single_blocks):
            b.reload_model_from_state_dict("single_transformer_blocks.%d." % j, sd, device)
        self._w = w

    def _bin_files(self):
        D = self.dim
        files = [("x_embedder.weight", (D, self.in_ch), "T"), ("x_embedder.bias", (D,), "T"),
                 ("context_embedder.weight", (D, self.joint_dim), "T"), ("context_embedder.bias", (D,), "T"),
                 ("proj_out.weight", (self.in_ch, D), "T"), ("proj_out.bias", (self.in_ch,), "T"),
                 ("norm_out.linear.weight", (2 * D, D), "T"), ("norm_out.linear.bias", (2 * D,), "T")]
        files += _mlp_files("time_text_embed.timestep_embedder.", 256, D) + _mlp_files("time_text_embed.guidance_embedder.", 256, D)
        files += _mlp_files("time_text_embed.text_embedder.", self.pooled_dim, D)
        for i, b in enumerate(self.double_blocks):
            files += [("transformer_blocks.%d.%s" % (i, k), shape, kind) for k, shape, kind in b._bin_files()]
        for j, b in enumerate(self.single_blocks):
            files += [("single_transformer_blocks.%d.%s" % (j, k), shape, kind) for k, shape, kind in b._bin_files()]
        return files

    def reload_transformer_model(self, model_path, model_dtype):
        """FluxTransformer2DModelWeight<T>::loadWeights (FluxTransformer2DModelWeight.cc:239-275): raw `<model_path><key>.bin`
        files, `model_dtype` "fp32" or "fp16" being the file type of the 16-bit tensors."""
        if len(model_path) > 0 and model_path[-1] != "/":
            model_path += "/"
        self.reload_transformer_model_from_state_dict(_state_dict_from_bin(model_path, model_dtype, self._bin_files()), "cuda")

    def _lora_table(self):
        """FluxTransformer2DModelWeight.cc:34-97,160-175: blocks under `transformer_blocks_<i>` / `single_transformer_blocks_<j>`,
        the embedders under `time_text_embed`, then `norm_out`, `x_embedder`, `context_embedder`, `proj_out`."""
        if self._w is None:
            raise RuntimeError("weights not loaded")
        w = self._w
        table = {"x_embedder": w["x_embedder"], "context_embedder": w["context_embedder"], "proj_out": w["proj_out"],
                 "norm_out": {"linear": w["norm_out"]},
                 "time_text_embed": {n: w[n].lora_table() for n in ("timestep_embedder", "guidance_embedder", "text_embedder")}}
        for i, b in enumerate(self.double_blocks):
            table["transformer_blocks_%d" % i] = b._lora_table()
        for j, b in enumerate(self.single_blocks):
            table["single_transformer_blocks_%d" % j] = b._lora_table()
        return table

    def load_lora_by_name(self, names, weight, scale):
        _load_lora_by_name(self._lora_table(), list(names), weight, float(scale))

    def clear_lora(self):
        _clear_lora(self._lora_table())

    def transformer_forward(self, hidden_states, encoder_hidden_states, rope_emb, pooled_projection, timestep, guidance,
                            controlnet_block_samples=None, controlnet_single_block_samples=None, controlnet_blocks_repeat=False):
        """hidden_states [B, S, input_channels], encoder_hidden_states [B, E, joint_attention_dim], rope_emb over the E + S
        joint sequence (text first), pooled_projection [B, pooled_projection_dim]; timestep and guidance are Python floats
        (the reference takes doubles).  Returns [B, S, input_channels]."""
        if self._w is None:
            raise RuntimeError("weights not loaded")
        for t in (hidden_states, encoder_hidden_states, rope_emb, pooled_projection):
            if not (t.is_cuda and t.is_contiguous() and t.dtype == self.dtype):
                raise RuntimeError("inputs must be contiguous CUDA tensors of the inference dtype")
        if controlnet_single_block_samples:
            raise RuntimeError("controlnet_single_block_samples currently needs to be 0")  # FluxTransformer2DModel.cc:252
        w, dt, dev = self._w, self.dtype, hidden_states.device
        B, S, _ = hidden_states.shape
        E, D = encoder_hidden_states.shape[1], self.dim
        if B != 1 and pooled_projection.shape[0] != B:
            raise RuntimeError("shape mismatch")

        # conditioning vector, SiLU'd as the blocks expect it (CombinedTimestepGuidanceTextProjEmbeddings, need_silu = true)
        t_emb = w["timestep_embedder"](time_projection(timestep, w["exponents"], dt))
        g_emb = w["guidance_embedder"](time_projection(guidance, w["exponents"], dt))
        p_emb = w["text_embedder"](pooled_projection)
        temb = torch.nn.functional.silu(((p_emb + g_emb) + t_emb)).contiguous()   # add3Tensor2dAndSilu: src1 + src2 + src3 in T

        h = torch.addmm(w["x_embedder"].b, hidden_states.view(B * S, -1), w["x_embedder"].w.t()).view(B, S, D)
        c = torch.addmm(w["context_embedder"].b, encoder_hidden_states.view(B * E, -1), w["context_embedder"].w.t()).view(B, E, D)

        # Every block's modulation linear depends on temb alone (an M = B matrix-vector product that streams 56-113 MB of
        # weights): all of them are issued on a second stream now, and each block waits only for its own, so that memory-bound
        # work overlaps the tensor-bound GEMMs of the blocks in front of it instead of standing between them.
        main = torch.cuda.current_stream()
        if self._side is None:
            self._side = torch.cuda.Stream()
        side = self._side if self.overlap_modulation else main
        side.wait_stream(main)
        mods = []
        with torch.cuda.stream(side):
            for block in self.double_blocks + self.single_blocks:
                mods.append((block.modulation(temb), side.record_event()))
        temb.record_stream(side)

        samples = list(controlnet_block_samples or [])
        interval = (self.n_double - 1) // len(samples) + 1 if samples else 0
        for i, block in enumerate(self.double_blocks):
            h, c = block.forward(h, c, rope_emb, temb, mods[i])
            if samples:
                res = samples[i % len(samples)] if controlnet_blocks_repeat else samples[i // interval]
                ops.invoke_load_lora(h, res.contiguous(), 1.0)

        x = torch.cat([c, h], dim=1)
        for j, block in enumerate(self.single_blocks):
            x = block.forward(x, rope_emb, temb, mods[self.n_double + j])
        main.wait_stream(side)
        h = x[:, E:].contiguous()

        # norm_out: AdaLayerNorm<T>(dim, 2, switch_scale = true): scale first, then shift (AdaLayerNorm.cc forward)
        msa = torch.addmm(w["norm_out"].b, temb, w["norm_out"].w.t())
        scale, shift = (t.contiguous() for t in msa.chunk(2, dim=1))
        normed = torch.empty_like(h)
        ops.invoke_layer_norm_with_shift_and_scale(normed, h, scale, shift, eps=1e-6)
        out = torch.addmm(w["proj_out"].b, normed.view(B * S, D), w["proj_out"].w.t())
        return out.view(B, S, self.in_ch)
