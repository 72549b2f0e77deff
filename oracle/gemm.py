"""Quantized GEMMs of the reference with their epilogues, restated on the CPU (test infrastructure).

Integer contractions are exact (done as fp32 BLAS products over K-chunks short
enough that every partial sum is an integer below 2**24, then summed in int64).
"""

import math

import torch

from . import quant as _q

F32 = torch.float32


def int_matmul_exact(a, b, chunk=1024):
    """Exact int32 C[m,n] = sum_k a[m,k]*b[n,k] for int8-range operands.

    |a|,|b| <= 128 so a chunk of 1024 products sums to at most 2**24: exact in fp32.
    """
    a = a.to(torch.int8) if a.dtype != torch.int8 else a
    m, k = a.shape
    acc = torch.zeros((m, b.shape[0]), dtype=torch.int64)
    for k0 in range(0, k, chunk):
        pa = a[:, k0:k0 + chunk].to(F32)
        pb = b[:, k0:k0 + chunk].to(F32)
        acc += (pa @ pb.t()).to(torch.int64)
    return acc.to(torch.int32)


def _round_to(v, dtype):
    return v.to(dtype)


# --------------------------------------------------------------------------- INT8 SmoothQuant W8A8
def int8_gemm_acc(qa, qw):
    """s8 x s8 -> s32 accumulators, A [M,K] row-major, W [N,K] (K contiguous):
    the contraction of CutlassInt8GemmRunner
    (src/lyradiff/kernels/cutlass_kernels/int8_gemm/int8_gemm_template.h:45-189)."""
    return int_matmul_exact(qa, qw)


def int8_gemm(qa, qw, alpha_col, alpha_row, out_dtype, per_token=False, bias=None, acc=None, residual=None):
    """C = T(float(acc) * (alpha_col[n] * alpha_row)), then bias added in T arithmetic.

    Scale order follows EpilogueVisitorPerRowPerCol
    (src/lyradiff/kernels/cutlass_extensions/include/cutlass_extensions/epilogue/threadblock/
    epilogue_per_row_per_col_scale.h:238-305): the two scales are multiplied first.
    The bias add follows the kernel that consumes the GEMM output in T precision
    (src/lyradiff/kernels/quant_kernels/ffn_kernels_int8.cu:126-129): y = T(T(acc*scale) + bias).
    alpha_row is fp32 [1] (per tensor) or [M] (per token).
    """
    if acc is None:
        acc = int8_gemm_acc(qa, qw)
    ar = alpha_row.to(F32).reshape(-1)
    ar = ar[:, None] if per_token else ar[0]
    scale = alpha_col.to(F32)[None, :] * ar
    y = _round_to(acc.to(F32) * scale, out_dtype)
    if residual is not None:
        # fusedBiasResidualAdd (src/lyradiff/kernels/basic_transformer/basic_transformer_kernels.cu:183-215):
        # src + residual + bias in T arithmetic, left to right
        y = _round_to(y.to(F32) + residual.to(F32), out_dtype)
    if bias is not None:
        y = _round_to(y.to(F32) + bias.to(F32)[None, :], out_dtype)
    return y


# --------------------------------------------------------------------------- FP8 e4m3
def gelu_tanh(v):
    """tanh-GELU in fp32 (src/lyradiff/kernels/activation_kernels.h:56-68), with an exact tanh."""
    return 0.5 * v * (1.0 + torch.tanh(0.7978845608028654 * (v + 0.044715 * v * v * v)))


def fp8_gemm(qx, qw, s_x, s_w, out_dtype=torch.bfloat16, bias=None, residual=None,
             alpha=1.0, beta=1.0, gelu=False):
    """Y[M,N] = T( epi( alpha*s_w*s_x * sum_k float(qw[n,k])*float(qx[m,k]) + beta*R + bias ) ).

    Follows cublasMMWrapper::GemmWithResidualAndBias for e4m3 operands
    (src/lyradiff/utils/cublasMMWrapper.cc:1104-1276): A/B scale pointers, fp32 compute,
    BIAS / GELU_BIAS / GELU epilogue, beta*Residual through the C operand (beta forced to 0
    without a residual).  The reference arithmetic is a closed library, so only tolerance
    parity is meaningful; the contraction here is carried in fp64.
    qx, qw are uint8 e4m3 codes.
    """
    x = _q.fp8_dequant(qx).double()
    w = _q.fp8_dequant(qw).double()
    acc = x @ w.t()
    sc = float(alpha) * float(s_w.reshape(-1)[0]) * float(s_x.reshape(-1)[0])
    v = acc * sc
    if residual is not None:
        v = v + float(beta) * residual.double()
    if bias is not None:
        v = v + bias.double()[None, :]
    if gelu:
        v = gelu_tanh(v)
    return v.to(F32).to(out_dtype)


# --------------------------------------------------------------------------- W4A4, group 64
def w4a4_group_partials(qa, qw, group=64):
    """Exact int32 partial products per K-group: p[g, m, n] = sum_{k in g} a[m,k]*w[n,k]."""
    m, k = qa.shape
    out = []
    for g in range(k // group):
        pa = qa[:, g * group:(g + 1) * group].to(F32)
        pw = qw[:, g * group:(g + 1) * group].to(F32)
        out.append((pa @ pw.t()).to(torch.int32))
    return out


def w4a4_gemm(qa, qw, sa, sb, out_dtype=torch.bfloat16, group=64, bias=None, gelu=False,
              residual=None, lora_act=None, lora_up=None, fma=True, round_each=False):
    """Grouped s4 GEMM with fp32 rescale.

    Follows w4a4_gemm (src/lyradiff/kernels/w4a4_gemm/w4a4_gemm.cu:473-507): for g in order,
    p = exact int32 dot over the group; acc += float(p) * sa[m,g] * sb[n,g] in fp32.  The source
    expression leaves the last multiply-add open to contraction, and the reference builds with
    nvcc's default -fmad=true, so the compiled arithmetic is t = fl(float(p)*sa);
    acc = fma(t, sb, acc) (one rounding); fma=True (default) restates that, fma=False rounds
    the second multiply and the add separately.  The two differ by at most one fp32 ulp per
    group.  LoRA-up (``:514-663``) adds
    sum_r bf16 lora_act[m,r] * bf16 lora_up[n,r] in fp32 after all groups.  The store is
    T(acc) (``:717``); bias / GELU-tanh / residual follow the standalone kernels that come
    next in the reference (src/lyradiff/kernels/flux_single_transformer_block/
    flux_single_transformer_kernels.cu:68-134) but are applied here in fp32 before the one
    rounding, which is the fused order this build uses; round_each=True instead rounds to T after
    the store and after each of those kernels, which is what the reference's separate launches give
    (T(acc) ``:717``; `add` of two T2 values in fusedBiasAndGelu / fusedBiasAndResidual rounds to T).
    qa [M,K], qw [N,K] unpacked int8 in [-8,7]; sa fp32 [M,K/g]; sb fp32|fp16 [N,K/g].
    """
    m, k = qa.shape
    n = qw.shape[0]
    acc = torch.zeros((m, n), dtype=F32)
    sa = sa.to(F32)
    sb = sb.to(F32)
    for g in range(k // group):
        pa = qa[:, g * group:(g + 1) * group].to(F32)
        pw = qw[:, g * group:(g + 1) * group].to(F32)
        p = pa @ pw.t()  # exact: |p| <= 64*64
        t = p * sa[:, g:g + 1]
        if fma:
            # t*sb is exact in fp64 (24+24 significand bits); one rounding to fp32 after the add
            acc = (t.double() * sb[None, :, g].double() + acc.double()).to(F32)
        else:
            acc = acc + t * sb[None, :, g]
    if lora_act is not None:
        # W4A4Gemm.cc:143 converts the fp32 down-projection to T before the low-rank MMA; the 32 products per
        # output are summed here in fp64 and added to the fp32 accumulator in one step
        a16 = lora_act.to(out_dtype if out_dtype != F32 else torch.bfloat16).double()
        acc = (acc.double() + a16 @ lora_up.double().t()).to(F32)
    rnd = (lambda t: t.to(out_dtype).to(F32)) if round_each else (lambda t: t)
    acc = rnd(acc)
    if bias is not None:
        acc = rnd(acc + bias.to(F32)[None, :])
    if gelu:
        acc = rnd(gelu_tanh(acc))
    if residual is not None:
        acc = acc + residual.to(F32)
    return acc.to(out_dtype)


def flops(m, n, k):
    return 2.0 * m * n * k


def gelu_tanh_scalar(v):
    return 0.5 * v * (1.0 + math.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3)))
