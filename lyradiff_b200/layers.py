"""Quantized-Linear layers over the C ABI: the host-side mirror of the reference's layer objects for this path.

Each class holds quantized weights and scales the way the reference's *Weight classes do, quantizes on load with the
device quantizers, owns a workspace for the quantized activation, and its forward() is one C-ABI call
(lyraq_*_forward).  torch supplies device memory and the stream; nothing is computed in torch.
"""

import torch

from . import _lib, ops

OP_LINEAR_INT8, OP_LINEAR_FP8, OP_LINEAR_W4A4, OP_LINEAR_W4A4_LORA = 3, 4, 5, 6


def _workspace(op, m, n, k, device, current):
    need = _lib.lib().lyraq_workspace_bytes(op, m, n, k)
    if current is None or current.numel() < need or current.device != device:
        current = torch.empty(max(need, 256), dtype=torch.uint8, device=device)
    return current


class Fp8Linear:
    """FP8 e4m3 linear of the FLUX blocks: weight quantized on load with a per-tensor amax/448 scale
    (MACROLoadFP8WeightFromCache, src/lyradiff/utils/common_macro_def.h:76-92), static activation scale,
    bias / GELU-tanh / residual fused into the GEMM epilogue."""

    def __init__(self, weight, bias, input_scale, gelu=False):
        n, k = weight.shape
        dev = weight.device
        self.n, self.k, self.gelu = n, k, gelu
        self.w_scale = torch.empty(1, dtype=torch.float32, device=dev)
        self.qweight = torch.empty(n, k, dtype=torch.uint8, device=dev)
        ops.weight_quant_fp8(self.qweight, self.w_scale, weight.contiguous())
        self.bias = None if bias is None else bias.contiguous()
        self.input_scale = input_scale.to(device=dev, dtype=torch.float32).reshape(1).contiguous()
        self._ws = None

    def forward(self, x, residual=None, beta=1.0, out=None):
        m = x.numel() // self.k
        x2 = x.reshape(m, self.k)
        y = out if out is not None else torch.empty(m, self.n, dtype=x.dtype, device=x.device)
        self._ws = _workspace(OP_LINEAR_FP8, m, self.n, self.k, x.device, self._ws)
        st = _lib.lib().lyraq_linear_fp8_forward(
            ops._p(y), ops._p(x2), ops._dt(x2), ops._p(self.input_scale), ops._p(self.qweight), ops._p(self.w_scale),
            ops._p(self.bias), ops._p(residual), float(beta), ops.EPI_GELU_TANH if self.gelu else ops.EPI_NONE, m, self.n,
            self.k, ops._p(self._ws), self._ws.numel(), ops._stream())
        _lib.check(st, "lyraq_linear_fp8_forward")
        return y.reshape(*x.shape[:-1], self.n)


class SmoothQuantLinear:
    """INT8 SmoothQuant W8A8 linear of the SDXL INT8 block: int8 weight + per-channel scale + smoothing vector
    (.weight_int8 / .weight_quant_scale / .pre_quant_scale / .input_quant_scale,
    src/lyradiff/layers/basic_transformer/BasicTransformerInt8BlockWeight.cc:249-288).  input_scale=None selects
    dynamic per-token activation scales."""

    def __init__(self, qweight, weight_scale, pre_quant_scale, bias=None, input_scale=None):
        self.n, self.k = qweight.shape
        self.qweight, self.w_scale, self.pre = qweight.contiguous(), weight_scale.contiguous(), pre_quant_scale
        self.bias, self.input_scale = bias, input_scale
        self._ws = None

    @classmethod
    def from_float(cls, weight, pre_quant_scale, bias=None, input_scale=None):
        """Quantizes a floating-point weight on the device as invokeGetINT8WeightScale does
        (src/lyradiff/kernels/quant_kernels/quant_kernels.cu:270-312)."""
        n, k = weight.shape
        qw = torch.empty(n, k, dtype=torch.int8, device=weight.device)
        sw = torch.empty(n, dtype=torch.float32, device=weight.device)
        ops.invoke_get_int8_weight_scale(sw, qw, weight.contiguous(), pre_quant_scale)
        return cls(qw, sw, pre_quant_scale, bias, input_scale)

    @staticmethod
    def bin_files(name, d_out, d_in, has_bias=True):
        """The raw files of one INT8 linear `name` (e.g. "ff.net.0.proj") under a block prefix, as the reference's loader
        reads them (MACROLoadLinearInt8WeightFromBin, src/lyradiff/utils/common_macro_def.h:51-59, used at
        layers/basic_transformer/BasicTransformerInt8BlockWeight.cc:249-288; written by the exporter,
        lyradiff/convert_model_scripts/convert_sd_quant_model.py:182-219): (suffix, element kind, shape)."""
        files = [(name + ".weight_int8.bin", "int8", (d_out, d_in)), (name + ".weight_quant_scale.bin", "fp32", (d_out,)),
                 (name + ".input_quant_scale.bin", "fp32", (1,)), (name + ".pre_quant_scale.bin", "fp32", (d_in,))]
        if has_bias:
            files.append((name + ".bias.bin", "model", (d_out,)))
        return files

    @classmethod
    def from_bin(cls, prefix, name, d_out, d_in, dtype=torch.float16, model_file_type="fp16", has_bias=True, device="cuda"):
        """Reads <prefix><name>.weight_int8.bin / .weight_quant_scale.bin / .input_quant_scale.bin / .pre_quant_scale.bin
        (+ .bias.bin in the model's file type, "fp32" or "fp16") and returns the linear with its static input scale.  A
        missing or short file raises; nothing is defaulted."""
        import numpy as np
        kinds = {"int8": np.int8, "fp32": np.float32, "model": {"fp32": np.float32, "fp16": np.float16}[model_file_type]}
        got = {}
        for fname, kind, shape in cls.bin_files(name, d_out, d_in, has_bias):
            path = prefix + fname
            count = int(np.prod(shape))
            arr = np.fromfile(path, dtype=kinds[kind])
            if arr.size != count:
                raise RuntimeError("%s holds %d elements, expected %d" % (path, arr.size, count))
            got[fname[len(name) + 1:-4]] = torch.from_numpy(arr.reshape(shape).copy())
        bias = got["bias"].to(dtype).to(device) if has_bias else None
        return cls(got["weight_int8"].to(device), got["weight_quant_scale"].to(device), got["pre_quant_scale"].to(device), bias,
                   got["input_quant_scale"].to(device))

    def forward(self, x, out=None):
        m = x.numel() // self.k
        x2 = x.reshape(m, self.k)
        y = out if out is not None else torch.empty(m, self.n, dtype=x.dtype, device=x.device)
        self._ws = _workspace(OP_LINEAR_INT8, m, self.n, self.k, x.device, self._ws)
        mode = ops.SCALE_PER_TOKEN_DYNAMIC if self.input_scale is None else ops.SCALE_PER_TENSOR
        st = _lib.lib().lyraq_linear_int8_forward(
            ops._p(y), ops._p(x2), ops._dt(x2), ops._p(self.pre), ops._p(self.input_scale), mode, ops._p(self.qweight),
            ops._p(self.w_scale), ops._p(self.bias), m, self.n, self.k, ops._p(self._ws), self._ws.numel(), ops._stream())
        _lib.check(st, "lyraq_linear_int8_forward")
        return y.reshape(*x.shape[:-1], self.n)


class W4A4Gemm:
    """W4A4 group-64 linear: W4A4Gemm<T> / W4A4GemmWeight<T> (src/lyradiff/layers/w4a4_gemm_block/W4A4Gemm.cc:113-169,
    W4A4GemmWeight.h:8-45): packed int4 weight [n, k/2], group scales [n, k/64], smoothing vector, optional bias."""

    def __init__(self, packed_weight, weight_scale, smooth=None, bias=None, gelu=False, lora_down=None, lora_up=None,
                 round_each=False):
        self.n, self.k = packed_weight.shape[0], packed_weight.shape[1] * 2
        self.qweight, self.w_scale, self.smooth, self.bias, self.gelu = packed_weight, weight_scale, smooth, bias, gelu
        if (lora_down is None) != (lora_up is None):
            raise ValueError("lora_down [32, k] and lora_up [n, 32] come together")
        self.lora_down, self.lora_up = lora_down, lora_up
        # round_each: round after every epilogue step (the bits of the reference's GEMM + separate 16-bit kernels)
        self._epi = (ops.EPI_GELU_TANH if gelu else ops.EPI_NONE) | (ops.EPI_ROUND_EACH if round_each else 0)
        self._ws = None

    @classmethod
    def from_float(cls, weight, smooth=None, bias=None, gelu=False, scale_dtype=torch.float16, lora_down=None, lora_up=None):
        n, k = weight.shape
        qw = torch.empty(n, k // 2, dtype=torch.uint8, device=weight.device)
        sw = torch.empty(n, k // 64, dtype=scale_dtype, device=weight.device)
        ops.weight_quant_int4_g64(qw, sw, weight.contiguous())
        return cls(qw, sw, smooth, bias, gelu, lora_down, lora_up)

    def forward(self, x, residual=None, out=None):
        m = x.numel() // self.k
        x2 = x.reshape(m, self.k)
        y = out if out is not None else torch.empty(m, self.n, dtype=x.dtype, device=x.device)
        if self.lora_down is not None:
            self._ws = _workspace(OP_LINEAR_W4A4_LORA, m, self.n, self.k, x.device, self._ws)
            st = _lib.lib().lyraq_w4a4_lora_forward(
                ops._p(y), ops._p(x2), ops._dt(x2), ops._p(self.smooth), ops._p(self.qweight), ops._p(self.w_scale),
                ops._dt(self.w_scale), ops._p(self.lora_down), ops._p(self.lora_up), ops._p(self.bias), ops._p(residual),
                self._epi, m, self.n, self.k, ops._p(self._ws), self._ws.numel(), ops._stream())
            _lib.check(st, "lyraq_w4a4_lora_forward")
            return y.reshape(*x.shape[:-1], self.n)
        self._ws = _workspace(OP_LINEAR_W4A4, m, self.n, self.k, x.device, self._ws)
        st = _lib.lib().lyraq_w4a4_forward(
            ops._p(y), ops._p(x2), ops._dt(x2), ops._p(self.smooth), ops._p(self.qweight), ops._p(self.w_scale),
            ops._dt(self.w_scale), ops._p(self.bias), ops._p(residual), self._epi, m,
            self.n, self.k, ops._p(self._ws), self._ws.numel(), ops._stream())
        _lib.check(st, "lyraq_w4a4_forward")
        return y.reshape(*x.shape[:-1], self.n)
