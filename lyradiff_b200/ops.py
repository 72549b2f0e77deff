"""Host-side mirror of the reference's layer-level functions over the C ABI.

Each function has the name, argument meaning and error behaviour of the reference function it
replaces (cited per function), takes torch CUDA tensors where the reference takes raw device
pointers, runs on torch's current stream and never synchronises.  torch is used only for device
memory and streams; all arithmetic happens in liblyraq.so.
"""

import torch

from . import _lib

F16, BF16, F32, S32, E4M3 = 0, 1, 2, 3, 4
SCALE_PER_TENSOR, SCALE_PER_TOKEN, SCALE_PER_TOKEN_DYNAMIC = 0, 1, 2
EPI_NONE, EPI_GELU_TANH, EPI_ROUND_EACH = 0, 1, 2

_DTYPES = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32, torch.int32: S32}


def _dt(t):
    try:
        return _DTYPES[t.dtype if isinstance(t, torch.Tensor) else t]
    except KeyError:
        raise TypeError("unsupported dtype %s" % (t.dtype if isinstance(t, torch.Tensor) else t))


def _p(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("expected a CUDA tensor")
    if not t.is_contiguous():
        raise ValueError("expected a contiguous tensor")
    return t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def last_status():
    """Synchronises the current stream and returns (status, detail) of the device status word."""
    import ctypes
    d = ctypes.c_uint32(0)
    st = _lib.lib().lyraq_last_status(_stream(), ctypes.byref(d))
    return st, d.value


# ----------------------------------------------------------------------------- quantizers
def invoke_sq_input_quant(dst, src, pre_quant_scale, input_quant_scale, per_token=False, dynamic=False):
    """invokeSqInputQuant<T> (src/lyradiff/kernels/quant_kernels/quant_kernels.h:9-17).
    src [..., dim] fp16/bf16 -> dst int8 same shape.  `dynamic` computes per-token scales into input_quant_scale."""
    dim = src.shape[-1]
    rows = src.numel() // dim
    mode = SCALE_PER_TOKEN_DYNAMIC if dynamic else (SCALE_PER_TOKEN if per_token else SCALE_PER_TENSOR)
    st = _lib.lib().lyraq_quant_int8(_p(dst), _p(src), _dt(src), _p(pre_quant_scale), _p(input_quant_scale), mode, rows,
                                     dim, _stream())
    _lib.check(st, "lyraq_quant_int8")
    return dst


def invoke_cuda_d2d_scale_cpy_convert(dst, src, scale, invert_scale=True):
    """invokeCudaD2DScaleCpyConvert<Tin, __nv_fp8_e4m3> (src/lyradiff/utils/memory_utils.h:74).  dst: uint8 e4m3 codes."""
    st = _lib.lib().lyraq_quant_fp8(_p(dst), _p(src), _dt(src), _p(scale), 1 if invert_scale else 0, src.numel(), _stream())
    _lib.check(st, "lyraq_quant_fp8")
    return dst


def invoke_get_fp8_weight_scale(scale, weight):
    """invokeGetFP8WeightScale (src/lyradiff/kernels/lora/load_lora.cu:109-113): scale = max(scale, max|w|/448)."""
    st = _lib.lib().lyraq_fp8_amax_scale(_p(scale), _p(weight), _dt(weight), weight.numel(), _stream())
    _lib.check(st, "lyraq_fp8_amax_scale")
    return scale


def weight_quant_fp8(qw, scale, weight):
    """MACROLoadFP8WeightFromCache (src/lyradiff/utils/common_macro_def.h:76-92) in one call: scale = max|w|/448 and
    qw = e4m3(w / scale), stream-ordered."""
    st = _lib.lib().lyraq_weight_quant_fp8(_p(qw), _p(scale), _p(weight), _dt(weight), weight.numel(), _stream())
    _lib.check(st, "lyraq_weight_quant_fp8")
    return qw, scale


def invoke_get_int8_weight_scale(new_weight_scale, quantized_weight, weight, pre_quant_scale):
    """invokeGetINT8WeightScale<T> (src/lyradiff/kernels/quant_kernels/quant_kernels.cu:270-312)."""
    d_out, d_in = weight.shape
    st = _lib.lib().lyraq_weight_quant_int8(_p(new_weight_scale), _p(quantized_weight), _p(weight), _dt(weight),
                                            _p(pre_quant_scale), d_out, d_in, _stream())
    _lib.check(st, "lyraq_weight_quant_int8")
    return quantized_weight, new_weight_scale


def invoke_fused_quantize_and_lora_down_simple(lora_act, q, q_scale, x, lora_down, smooth):
    """invokeFusedQuantizeAndLoraDownSimple (src/lyradiff/kernels/w4a4_gemm/w4a4_gemm.h:6-17).
    x [m,k] -> q uint8 [m,k/2], q_scale fp32 [m,k/64]; lora_act fp32 [m,32] if lora_down [32,k] is given."""
    m, k = x.shape
    st = _lib.lib().lyraq_quant_int4_g64(_p(q), _p(q_scale), _p(lora_act), _p(x), _dt(x), _p(smooth), _p(lora_down), m, k,
                                         _stream())
    _lib.check(st, "lyraq_quant_int4_g64")
    return q, q_scale


def weight_quant_int4_g64(qw, w_scale, w):
    """INT4 group-64 weight quantize into the W4A4GemmWeight layout
    (src/lyradiff/layers/w4a4_gemm_block/W4A4GemmWeight.h:8-45)."""
    n, k = w.shape
    st = _lib.lib().lyraq_weight_quant_int4_g64(_p(qw), _p(w_scale), _dt(w_scale), _p(w), _dt(w), n, k, _stream())
    _lib.check(st, "lyraq_weight_quant_int4_g64")
    return qw, w_scale


# ----------------------------------------------------------------------------- fused producers
def invoke_layer_norm_with_shift_and_scale(dst, src, scale, shift, eps=1e-6, q8=None, q8_scale=None, qf8=None,
                                           f8_scale=None, pre_quant_scale=None):
    """invokeLayerNormWithShiftAndScale<T> (src/lyradiff/kernels/norms/layer_norm.h:19) with the quantize pass fused in.
    src [B,S,D]; scale, shift [B,D]; dst may be None when only quantized outputs are wanted."""
    b, s, d = src.shape
    st = _lib.lib().lyraq_adaln_quant(_p(dst), _p(q8), _p(q8_scale), _p(qf8), _p(f8_scale), _p(src), _p(scale), _p(shift),
                                      _dt(src), _p(pre_quant_scale), b, s, d, float(eps), _stream())
    _lib.check(st, "lyraq_adaln_quant")
    return dst


def adaln_quant_fp8x2(dst, qa, scale_a, qb, scale_b, src, scale, shift, eps=1e-6):
    """AdaLN modulation with two e4m3 outputs (two consumers with their own input scales) in one pass
    (lyraq_adaln_quant_fp8x2); dst (16-bit) may be None."""
    b, s, d = src.shape
    st = _lib.lib().lyraq_adaln_quant_fp8x2(_p(dst), _p(qa), _p(scale_a), _p(qb), _p(scale_b), _p(src), _p(scale), _p(shift),
                                            _dt(src), b, s, d, float(eps), _stream())
    _lib.check(st, "lyraq_adaln_quant_fp8x2")
    return qa, qb


def invoke_layer_norm_int8o(dst, src, gamma, beta, pre_quant_scale, input_quant_scale, eps=1e-5, residual=None,
                            bias=None, sum_out=None):
    """invokeLayerNormInt8O<T> / invokeFusedResidualBiasLayerNormInt8O<T>
    (src/lyradiff/kernels/quant_kernels/layer_norm_int8.h:9-38)."""
    dim = src.shape[-1]
    rows = src.numel() // dim
    st = _lib.lib().lyraq_ln_quant_int8(_p(dst), _p(sum_out), _p(src), _p(residual), _p(bias), _p(gamma), _p(beta),
                                        _dt(src), _p(pre_quant_scale), _p(input_quant_scale), rows, dim, float(eps),
                                        _stream())
    _lib.check(st, "lyraq_ln_quant_int8")
    return dst


def invoke_fused_add_bias_geglu_int8o(dst, hidden_states, bias, pre_quant_scale, input_quant_scale):
    """invokeFusedAddBiasGegluInt8O<T> (src/lyradiff/kernels/quant_kernels/ffn_kernels_int8.h:13-21).
    hidden_states [..., 2*dim] -> dst int8 [..., dim]."""
    dim = hidden_states.shape[-1] // 2
    rows = hidden_states.numel() // (2 * dim)
    st = _lib.lib().lyraq_geglu_quant_int8(_p(dst), _p(hidden_states), _p(bias), _dt(hidden_states), _p(pre_quant_scale),
                                           _p(input_quant_scale), rows, dim, _stream())
    _lib.check(st, "lyraq_geglu_quant_int8")
    return dst


# ----------------------------------------------------------------------------- GEMMs
def run_gemm_int8(A, B, alpha_col, alpha_row, C, bias=None, per_token=False, workspace=None, residual=None):
    """cublasMMWrapper::runGemmInt8 (src/lyradiff/utils/cublasMMWrapper.h:368-385): C[m,n] from A int8 [m,k], B int8 [n,k].
    C dtype fp16/bf16/fp32 (dequantized) or int32 (raw accumulators).  `residual` [m,n] fuses the invokeFusedBiasResidualAdd
    that follows the SDXL feed-forward output linear (BasicTransformerInt8Block.cc:824-845)."""
    m, k = A.shape
    n = B.shape[0]
    if B.shape[1] != k or tuple(C.shape) != (m, n):
        raise ValueError("shape mismatch")
    ws = 0 if workspace is None else workspace.numel() * workspace.element_size()
    if residual is not None:
        if tuple(residual.shape) != (m, n) or residual.dtype != C.dtype:
            raise ValueError("residual must have the shape and dtype of C")
        st = _lib.lib().lyraq_gemm_int8_residual(_p(A), _p(B), _p(alpha_col), _p(alpha_row),
                                                 SCALE_PER_TOKEN if per_token else SCALE_PER_TENSOR, _p(C), _dt(C), _p(bias),
                                                 _p(residual), m, n, k, _p(workspace), ws, _stream())
        _lib.check(st, "lyraq_gemm_int8_residual")
        return C
    st = _lib.lib().lyraq_gemm_int8(_p(A), _p(B), _p(alpha_col), _p(alpha_row),
                                    SCALE_PER_TOKEN if per_token else SCALE_PER_TENSOR, _p(C), _dt(C), _p(bias), m, n, k,
                                    _p(workspace), ws, _stream())
    _lib.check(st, "lyraq_gemm_int8")
    return C


def gemm_with_residual_and_bias_fp8(W, w_scale, X, x_scale, Y, bias=None, residual=None, alpha=1.0, beta=1.0,
                                    is_gelu=False):
    """cublasMMWrapper::GemmWithResidualAndBias for e4m3 (src/lyradiff/utils/cublasMMWrapper.h:300-317), in the reference's
    argument order (weight first): Y[m,n] = epi(alpha*s_w*s_x * X[m,k] W[n,k]^T + beta*R + bias)."""
    m, k = X.shape
    n = W.shape[0]
    if W.shape[1] != k or tuple(Y.shape) != (m, n):
        raise ValueError("shape mismatch")
    st = _lib.lib().lyraq_gemm_fp8(_p(X), _p(x_scale), _p(W), _p(w_scale), _p(Y), _dt(Y), _p(bias), _p(residual),
                                   float(alpha), float(beta), EPI_GELU_TANH if is_gelu else EPI_NONE, m, n, k, None, 0,
                                   _stream())
    _lib.check(st, "lyraq_gemm_fp8")
    return Y


def gemm_fp8_qk_rope(W, w_scale, X, x_scale, Y, qk_scale, rope_emb, heads, head_dim, bias=None, eps=1e-6):
    """The to_qkv FP8 GEMM with invokeFusedRmsNormAndRope (src/lyradiff/kernels/rope/flux_apply_rope.h:20-30) fused into its
    epilogue: Y [m, 3*heads*head_dim] (rows may be a window of a taller, equally wide tensor) gets the projection with q and k
    heads normalised and rotated; rope_emb holds the rotations of exactly these m rows.  Same bits as
    gemm_with_residual_and_bias_fp8 followed by invoke_fused_rmsnorm_and_rope in place."""
    m, k = X.shape
    n = W.shape[0]
    if W.shape[1] != k or tuple(Y.shape) != (m, n) or Y.stride(1) != 1 or rope_emb.numel() != m * head_dim * 2:
        raise ValueError("shape mismatch")
    st = _lib.lib().lyraq_gemm_fp8_qk_rope(_p(X), _p(x_scale), _p(W), _p(w_scale), _p(Y), Y.stride(0), _dt(Y), _p(bias), _p(qk_scale),
                                           _p(rope_emb), heads, head_dim, float(eps), m, n, k, _stream())
    _lib.check(st, "lyraq_gemm_fp8_qk_rope")
    return Y


def invoke_fused_rmsnorm_and_rope(out, qkv, scale, rope_emb, eps, batch, seq_len, heads, head_dim):
    """invokeFusedRmsNormAndRope<T> (src/lyradiff/kernels/rope/flux_apply_rope.h:20-30): qkv [batch, seq, 3*heads*head_dim]
    packed q|k|v, scale [2*head_dim], rope_emb [batch, seq, head_dim/2, 2, 2]; out may be qkv itself."""
    st = _lib.lib().lyraq_rmsnorm_rope(_p(out), _p(qkv), _p(scale), _p(rope_emb), _dt(qkv), float(eps), batch, seq_len, heads,
                                       head_dim, _stream())
    _lib.check(st, "lyraq_rmsnorm_rope")
    return out


def flash_attention(qkv, batch, seq_len, heads, head_dim, out=None, out_scale=None, col0=0, out2=None, out2_scale=None,
                    col0_2=0, split=None, softmax_scale=None):
    """FlashAttention2Layer<T>::forward (src/lyradiff/layers/flash_attn2/flash_attn2.cu:59-118) on the packed projection
    qkv [batch * seq_len, 3 * heads * head_dim].  out: [batch * rows, ld] of qkv's type, or uint8 (e4m3 codes, with
    out_scale) -- columns col0 .. col0 + heads * head_dim are written; created as a 16-bit [batch * seq_len, heads *
    head_dim] tensor when omitted.  With out2 / split the rows from `split` on go to out2 (see lyraq_attention)."""
    width = heads * head_dim
    if out is None:
        out = torch.empty(batch * seq_len, width, dtype=qkv.dtype, device=qkv.device)
    e4m3 = out.dtype == torch.uint8
    if split is None:
        split = seq_len
    if softmax_scale is None:
        softmax_scale = float(head_dim) ** -0.5
    esz = 1 if e4m3 else 2
    p1 = out.data_ptr() + col0 * esz
    p2 = None if out2 is None else out2.data_ptr() + col0_2 * esz
    if not out.is_contiguous() or (out2 is not None and not out2.is_contiguous()):
        raise ValueError("expected contiguous outputs")
    st = _lib.lib().lyraq_attention(p1, E4M3 if e4m3 else _dt(qkv), out.shape[-1], _p(out_scale), p2,
                                    0 if out2 is None else out2.shape[-1], _p(out2_scale), split, _p(qkv), _dt(qkv), batch,
                                    seq_len, heads, head_dim, float(softmax_scale), _stream())
    _lib.check(st, "lyraq_attention")
    return out


def quant_fp8_into_columns(dst, col0, src, scale):
    """e4m3 quantize of src [rows, cols] into dst[:, col0:col0+cols] (dst uint8 [rows, ld], contiguous)."""
    rows, cols = src.shape
    if dst.shape[0] != rows or col0 + cols > dst.shape[1]:
        raise ValueError("shape mismatch")
    st = _lib.lib().lyraq_quant_fp8_2d(dst.data_ptr() + col0, dst.shape[1], _p(src), _dt(src), _p(scale), rows, cols, _stream())
    _lib.check(st, "lyraq_quant_fp8_2d")
    return dst


def invoke_fused_gate_and_residual(out, y, gate, residual):
    """invokeFusedGateAndResidual<T> (flux_single_transformer_kernels.cu:152-160): out = y * gate[b] + residual."""
    b, s, d = y.shape
    st = _lib.lib().lyraq_gate_residual(_p(out), _p(y), _p(gate), _p(residual), _dt(y), b, s, d, _stream())
    _lib.check(st, "lyraq_gate_residual")
    return out


def invoke_load_lora(weight, lora, alpha):
    """invokeLoadLora<T> (src/lyradiff/kernels/lora/load_lora.h): weight += lora * alpha in place, in the weight's own 16-bit
    arithmetic (both steps rounded)."""
    if weight.shape != lora.shape or weight.dtype != lora.dtype or not (weight.is_contiguous() and lora.is_contiguous()):
        raise ValueError("weight and lora must be contiguous tensors of one shape and dtype")
    st = _lib.lib().lyraq_load_lora(_p(weight), _p(lora), _dt(weight), float(alpha), weight.numel(), _stream())
    _lib.check(st, "lyraq_load_lora")
    return weight


def gemm_fp8_gate_residual(W, w_scale, X, x_scale, Y, gate, residual, rows_per_batch, bias=None):
    """FP8 GEMM + invokeFusedGateAndResidual in one launch (lyraq_gemm_fp8_gate): Y = (X W^T * s + bias) * gate[b] + residual,
    rounded to Y's dtype after every step.  Returns False (nothing launched) when the shape cannot be fused."""
    m, k = X.shape
    n = W.shape[0]
    if W.shape[1] != k or tuple(Y.shape) != (m, n):
        raise ValueError("shape mismatch")
    if m > rows_per_batch and rows_per_batch % 256 != 0:
        return False
    st = _lib.lib().lyraq_gemm_fp8_gate(_p(X), _p(x_scale), _p(W), _p(w_scale), _p(Y), _dt(Y), _p(bias), _p(gate), _p(residual),
                                        rows_per_batch, m, n, k, None, 0, _stream())
    _lib.check(st, "lyraq_gemm_fp8_gate")
    return True


def gemm_fp8_quant_into_columns(W, w_scale, X, x_scale, dst, col0, y_scale, dtype, bias=None, is_gelu=False):
    """FP8 GEMM whose e4m3 result lands in dst[:, col0:col0+n] (lyraq_gemm_fp8_quant_ld)."""
    m, k = X.shape
    n = W.shape[0]
    if W.shape[1] != k or dst.shape[0] != m or col0 + n > dst.shape[1]:
        raise ValueError("shape mismatch")
    st = _lib.lib().lyraq_gemm_fp8_quant_ld(_p(X), _p(x_scale), _p(W), _p(w_scale), dst.data_ptr() + col0, dst.shape[1],
                                            _p(y_scale), _dt(dtype), _p(bias), None, 1.0, 0.0,
                                            EPI_GELU_TANH if is_gelu else EPI_NONE, m, n, k, None, 0, _stream())
    _lib.check(st, "lyraq_gemm_fp8_quant_ld")
    return dst


def gemm_fp8_quant_out(W, w_scale, X, x_scale, Yq, y_scale, dtype, bias=None, residual=None, alpha=1.0, beta=1.0, is_gelu=False):
    """FP8 GEMM whose epilogue also quantizes the result for the next FP8 linear (lyraq_gemm_fp8_quant): Yq uint8 e4m3 codes of
    T(epi(...)) / y_scale; `dtype` is the torch dtype T of bias / residual.  Fuses GemmWithResidualAndBias + GELU kernel +
    invokeCudaD2DScaleCpyConvert (FluxSingleTransformerFP8Block.cc:227-281)."""
    m, k = X.shape
    n = W.shape[0]
    if W.shape[1] != k or tuple(Yq.shape) != (m, n):
        raise ValueError("shape mismatch")
    st = _lib.lib().lyraq_gemm_fp8_quant(_p(X), _p(x_scale), _p(W), _p(w_scale), _p(Yq), _p(y_scale), _dt(dtype), _p(bias),
                                         _p(residual), float(alpha), float(beta), EPI_GELU_TANH if is_gelu else EPI_NONE, m, n, k,
                                         None, 0, _stream())
    _lib.check(st, "lyraq_gemm_fp8_quant")
    return Yq


def invoke_fused_w4a4_gemm_and_lora_up(D, A, B, lora_act, lora_up, sa, sb, bias=None, residual=None, is_gelu=False,
                                       round_each=False):
    """invokeFusedW4A4GemmAndLoraUp (src/lyradiff/kernels/w4a4_gemm/w4a4_gemm.h:19-30) with the bias / GELU / residual
    kernels that follow it fused in.  A uint8 [m,k/2], B uint8 [n,k/2], sa fp32 [m,k/64], sb fp32|fp16 [n,k/64];
    lora_act [m,32] fp32 (as the quantizer wrote it) or already of D's dtype, lora_up [n,32] of D's dtype.
    round_each: round to D's dtype after every epilogue step, as the reference's separate kernels do."""
    m, kh = A.shape
    n = B.shape[0]
    k = kh * 2
    if B.shape[1] != kh or tuple(D.shape) != (m, n):
        raise ValueError("shape mismatch")
    st = _lib.lib().lyraq_gemm_w4a4(_p(A), _p(B), _p(sa), _p(sb), _dt(sb), _p(D), _dt(D), _p(lora_act),
                                    F32 if lora_act is None else _dt(lora_act), _p(lora_up),
                                    _p(bias), _p(residual),
                                    (EPI_GELU_TANH if is_gelu else EPI_NONE) | (EPI_ROUND_EACH if round_each else 0), m, n, k,
                                    None, 0, _stream())
    _lib.check(st, "lyraq_gemm_w4a4")
    return D
