"""Generates the committed golden vectors under tests/golden/ from the CPU oracle.

    python tests/golden/make_golden.py

The reference ships no golden vectors or known-answer tests for this path and cannot be built
or run offline (no GPU, un-vendored CUTLASS), so these files pin the ORACLE against regressions;
they are small seeded cases (a few KB each).  16-bit float tensors are stored as their uint16 bit
patterns (key suffix `_bits16`, dtype recorded under `<name>_dtype`).
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from oracle import gemm, norms, quant, workloads  # noqa: E402


def put(d, name, t):
    if isinstance(t, torch.Tensor) and t.dtype in (torch.float16, torch.bfloat16):
        d[name + "_bits16"] = t.contiguous().view(torch.int16).numpy().view(np.uint16)
        d[name + "_dtype"] = np.array(str(t.dtype))
    elif isinstance(t, torch.Tensor):
        d[name] = t.contiguous().numpy()
    else:
        d[name] = np.asarray(t)


def get(z, name):
    """Inverse of put(): returns a torch tensor."""
    if name in z:
        return torch.from_numpy(np.array(z[name]))
    bits = torch.from_numpy(np.array(z[name + "_bits16"]).view(np.int16))
    dt = {"torch.float16": torch.float16, "torch.bfloat16": torch.bfloat16}[str(z[name + "_dtype"])]
    return bits.view(dt)


def case_int8():
    wl = workloads.int8_smoothquant_linear(m=48, k=64, n=40, seed=11)
    d = {}
    qa, sa = quant.sq_input_quant_dynamic(wl["x"], wl["pre"])
    static = torch.tensor([0.05], dtype=torch.float32)
    q_static = quant.sq_input_quant(wl["x"], wl["pre"], static)
    acc = gemm.int8_gemm_acc(qa, wl["qw"])
    y = gemm.int8_gemm(qa, wl["qw"], wl["s_w"], sa, torch.float16, per_token=True, bias=wl["bias"], acc=acc)
    for k in ("x", "w", "bias", "pre", "qw", "s_w"):
        put(d, k, wl[k])
    put(d, "qa", qa); put(d, "sa", sa); put(d, "static_scale", static); put(d, "q_static", q_static)
    put(d, "acc", acc); put(d, "y", y)
    return d


def case_fp8():
    f = workloads.fp8_linear(40, 64, 48, seed=12, with_residual=True)
    d = {}
    for k in ("x", "w", "bias", "residual", "s_x", "s_w", "qx", "qw"):
        put(d, k, f[k])
    put(d, "y_plain", gemm.fp8_gemm(f["qx"], f["qw"], f["s_x"], f["s_w"], bias=f["bias"]))
    put(d, "y_gelu", gemm.fp8_gemm(f["qx"], f["qw"], f["s_x"], f["s_w"], bias=f["bias"], gelu=True))
    put(d, "y_residual", gemm.fp8_gemm(f["qx"], f["qw"], f["s_x"], f["s_w"], bias=f["bias"], residual=f["residual"]))
    return d


def case_w4a4():
    w = workloads.w4a4_linear(m=24, k=128, n=40, seed=13, smooth_nontrivial=True, scale_dtype=torch.float32)
    d = {}
    pa, sa, qa = quant.int4_quant_g64(w["x"], w["smooth"])
    for k in ("x", "w", "smooth", "packed_w", "s_w", "qw"):
        put(d, k, w[k])
    put(d, "packed_a", pa); put(d, "sa", sa); put(d, "qa", qa)
    put(d, "y_bf16", gemm.w4a4_gemm(qa, w["qw"], sa, w["s_w"]))
    put(d, "y_f32", gemm.w4a4_gemm(qa, w["qw"], sa, w["s_w"], out_dtype=torch.float32))
    return d


def case_adaln():
    a = workloads.adaln_input(b=2, s=5, d=128, seed=14)
    f8 = torch.tensor([0.02], dtype=torch.float32)
    o = norms.adaln_quant(a["x"], a["scale"], a["shift"], fp8_scale=f8)
    d = {}
    for k in ("x", "scale", "shift"):
        put(d, k, a[k])
    put(d, "f8_scale", f8)
    for k in ("y", "q8", "s8", "qf8"):
        put(d, k, o[k])
    return d


def case_ln_geglu():
    g = torch.Generator().manual_seed(15)
    rows, dim = 6, 64
    x = torch.randn(rows, dim, generator=g).half()
    res = torch.randn(rows, dim, generator=g).half()
    bias = (torch.randn(dim, generator=g) * 0.1).half()
    gamma = (1.0 + 0.1 * torch.randn(dim, generator=g)).half()
    beta = (0.1 * torch.randn(dim, generator=g)).half()
    pre = (0.5 + torch.rand(dim, generator=g)).float()
    s = torch.tensor([0.03], dtype=torch.float32)
    q_ln, _ = norms.layernorm_int8(x, gamma, beta, pre, s)
    q_rln, hsum = norms.layernorm_int8(x, gamma, beta, pre, s, residual=res, bias=bias)
    h = torch.randn(rows, 2 * dim, generator=g).half()
    b2 = (torch.randn(2 * dim, generator=g) * 0.1).half()
    q_geglu = norms.geglu_int8(h, b2, pre, s)
    d = {}
    for k, v in (("x", x), ("residual", res), ("bias", bias), ("gamma", gamma), ("beta", beta), ("pre", pre),
                 ("scale", s), ("q_ln", q_ln), ("q_rln", q_rln), ("hsum", hsum), ("h", h), ("b2", b2),
                 ("q_geglu", q_geglu)):
        put(d, k, v)
    return d


CASES = {"int8": case_int8, "fp8": case_fp8, "w4a4": case_w4a4, "adaln": case_adaln, "ln_geglu": case_ln_geglu}


def main():
    torch.set_num_threads(1)
    for name, fn in CASES.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **fn())
        print("wrote", name)


if __name__ == "__main__":
    main()
