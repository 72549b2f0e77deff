"""GPU parity tests of the quantize / fused-producer kernels against the CPU oracle, through the C ABI."""

import pytest
import torch

from oracle import norms, quant, workloads
from tests.util import assert_bit_equal, check_status, cu, mismatch_fraction

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from lyradiff_b200 import ops as _ops
    return _ops


def _x(rows, dim, dtype, seed, outliers=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, dim, generator=g)
    if outliers and dim >= 20:
        x[:, torch.randperm(dim, generator=g)[: dim // 20]] *= 20.0
    pre = (0.25 + torch.rand(dim, generator=g)).float()
    return x.to(dtype), pre


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,dim", [(1, 8), (7, 64), (129, 640), (33, 3072), (5, 5120), (3, 16384), (260, 1280), (1, 640),
                                      (35, 320), (4099, 640)])
def test_int8_quant_all_scale_modes_bit_exact(ops, dtype, rows, dim):
    x, pre = _x(rows, dim, dtype, seed=rows * 31 + dim)
    xd, pred = cu(x), cu(pre)
    # static per-tensor scale (the reference's sqInputQuant)
    s = torch.tensor([0.043], dtype=torch.float32)
    q = torch.empty(rows, dim, dtype=torch.int8, device="cuda")
    ops.invoke_sq_input_quant(q, xd, pred, cu(s))
    assert_bit_equal(q, quant.sq_input_quant(x, pre, s), "static")
    # precomputed per-token scales (sqPerTokenInputQuant)
    st = (0.01 + torch.rand(rows)).float()
    ops.invoke_sq_input_quant(q, xd, pred, cu(st), per_token=True)
    assert_bit_equal(q, quant.sq_input_quant(x, pre, st, per_token=True), "per-token")
    # dynamic per-token
    sd = torch.empty(rows, dtype=torch.float32, device="cuda")
    ops.invoke_sq_input_quant(q, xd, pred, sd, dynamic=True)
    q_ref, s_ref = quant.sq_input_quant_dynamic(x, pre)
    assert_bit_equal(sd, s_ref, "dynamic scale")
    assert_bit_equal(q, q_ref, "dynamic q")
    # without the smoothing vector
    ops.invoke_sq_input_quant(q, xd, None, sd, dynamic=True)
    q_ref, s_ref = quant.sq_input_quant_dynamic(x, None)
    assert_bit_equal(sd, s_ref, "dynamic scale, no pre")
    assert_bit_equal(q, q_ref, "dynamic q, no pre")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,dim", [(1, 8), (3, 640), (129, 2560), (4099, 3072), (5, 16384)])
def test_int8_quant_special_kernels_give_the_row_kernel_bytes(ops, dtype, rows, dim):
    """With a static or a given per-token scale the quantize has no row statistic and runs as a flat kernel over 8-column
    vectors; with the dynamic scale rows of 320 / 640 / 1280 columns share a warp.  Either way the bytes (and the dynamic
    scales) must be those of the general row kernel."""
    from lyradiff_b200 import _lib

    x, pre = _x(rows, dim, dtype, seed=rows * 13 + dim)
    xd = cu(x)
    s = cu(torch.tensor([0.043], dtype=torch.float32))
    st = cu((0.01 + torch.rand(rows)).float())

    def run():
        out = []
        for smooth in (cu(pre), None):
            for kw, scale in (({}, s), ({"per_token": True}, st), ({"dynamic": True}, torch.zeros(rows, dtype=torch.float32, device="cuda"))):
                q = torch.full((rows, dim), 55, dtype=torch.int8, device="cuda")
                ops.invoke_sq_input_quant(q, xd, smooth, scale, **kw)
                check_status()
                out += [q.cpu(), scale.cpu().clone()]
        return out

    L = _lib.lib()
    special = run()
    assert L.lyraq_debug_set_special_row_kernels(0) == 0
    try:
        general = run()
    finally:
        L.lyraq_debug_set_special_row_kernels(1)
    for i, (a, b) in enumerate(zip(special, general)):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), i


def test_int8_quant_zero_rows_and_empty(ops):
    x = torch.zeros(4, 64, dtype=torch.float16)
    x[2] = torch.linspace(-2, 2, 64).half()
    q = torch.full((4, 64), 99, dtype=torch.int8, device="cuda")
    s = torch.empty(4, dtype=torch.float32, device="cuda")
    ops.invoke_sq_input_quant(q, cu(x), None, s, dynamic=True)
    q_ref, s_ref = quant.sq_input_quant_dynamic(x, None)
    assert_bit_equal(q, q_ref)
    assert_bit_equal(s, s_ref)
    assert s.cpu()[0].item() == 1.0
    # zero rows: nothing is launched, nothing fails
    ops.invoke_sq_input_quant(torch.empty(0, 64, dtype=torch.int8, device="cuda"),
                              torch.empty(0, 64, dtype=torch.float16, device="cuda"), None, s, dynamic=True)
    with pytest.raises(Exception):
        ops.invoke_sq_input_quant(q, cu(torch.zeros(4, 60, dtype=torch.float16)), None, s, dynamic=True)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n", [8, 1000, 4608 * 64 + 3, 1 << 20])
def test_fp8_quant_bit_exact(ops, dtype, n):
    g = torch.Generator().manual_seed(n)
    x = (torch.randn(n, generator=g) * 3.0).to(dtype)
    x[:: 97] *= 200.0  # exercise saturation to +-448
    s = torch.tensor([0.0371], dtype=torch.float32)
    q = torch.empty(n, dtype=torch.uint8, device="cuda")
    ops.invoke_cuda_d2d_scale_cpy_convert(q, cu(x), cu(s), invert_scale=True)
    assert_bit_equal(q, quant.fp8_quant(x, s, True), "invert")
    ops.invoke_cuda_d2d_scale_cpy_convert(q, cu(x), cu(s), invert_scale=False)
    assert_bit_equal(q, quant.fp8_quant(x, s, False), "direct")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fp8_weight_amax_scale_exact(ops, dtype):
    g = torch.Generator().manual_seed(5)
    w = (torch.randn(3072 * 96 + 5, generator=g) * 0.02).to(dtype)
    s = torch.zeros(1, dtype=torch.float32, device="cuda")
    ops.invoke_get_fp8_weight_scale(s, cu(w))
    assert_bit_equal(s, quant.fp8_amax_scale(w))
    # a second, smaller tensor leaves the running maximum alone
    ops.invoke_get_fp8_weight_scale(s, cu((w * 0.5).to(dtype)))
    assert_bit_equal(s, quant.fp8_amax_scale(w))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fp8_weight_quant_in_one_call(ops, dtype):
    """scale = max|w|/448 and e4m3(w/scale) from a stale scale buffer and a stale output, with no host step between."""
    g = torch.Generator().manual_seed(6)
    w = (torch.randn(640, 1288, generator=g) * 0.02).to(dtype)
    s = torch.full((1,), 123.0, dtype=torch.float32, device="cuda")
    q = torch.full((640, 1288), 0x7F, dtype=torch.uint8, device="cuda")
    ops.weight_quant_fp8(q, s, cu(w))
    want_s = quant.fp8_amax_scale(w)
    assert_bit_equal(s, want_s)
    assert_bit_equal(q, quant.fp8_quant(w, want_s, invert_scale=True))


def test_fp8_weight_quant_reads_its_scale_after_the_amax_kernel(ops):
    """The cast of lyraq_weight_quant_fp8 may start while the amax kernel in front of it still runs (programmatic
    dependent launch) and must read the scale only once that kernel has finished; an early read sees the zero the scale
    was reset to (every code saturates) or a partial maximum.  The window is narrow and depends on launch timing, so this
    loops over weights of several sizes copied from the host, as loading a model does."""
    g = torch.Generator().manual_seed(16)
    shapes = [(256, 256), (768, 256), (1536, 256), (256, 1024), (4096, 4096)]
    for i in range(60):
        n, k = shapes[i % len(shapes)]
        wi = cu((torch.randn(n, k, generator=g) * 0.02 * (0.5 + i % 7)).bfloat16())
        s = torch.full((1,), 1e30, dtype=torch.float32, device="cuda")
        q = torch.empty(n, k, dtype=torch.uint8, device="cuda")
        ops.weight_quant_fp8(q, s, wi)
        amax = float(wi.float().abs().max())
        assert abs(float(s) * 448.0 / amax - 1.0) < 1e-6
        codes = q.view(torch.float8_e4m3fn).float()
        assert float((codes.abs() >= 448.0).float().mean()) < 1e-2, "iteration %d: codes saturated" % i
        assert float((codes * float(s) - wi.float()).abs().max()) <= 0.07 * amax
    check_status()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,k", [(1, 64), (24, 128), (130, 3072), (5, 12288)])
def test_int4_g64_quant_bit_exact(ops, dtype, m, k):
    g = torch.Generator().manual_seed(m * 7 + k)
    x = torch.randn(m, k, generator=g).to(dtype)
    x[0, :64] = 0  # an all-zero group
    smooth = (0.5 + torch.rand(k, generator=g)).float()
    for sm in (smooth, None):
        q = torch.empty(m, k // 2, dtype=torch.uint8, device="cuda")
        s = torch.empty(m, k // 64, dtype=torch.float32, device="cuda")
        ops.invoke_fused_quantize_and_lora_down_simple(None, q, s, cu(x), None, cu(sm))
        p_ref, s_ref, _ = quant.int4_quant_g64(x, sm)
        assert_bit_equal(s, s_ref, "scales")
        assert_bit_equal(q, p_ref, "packed nibbles")


@pytest.mark.parametrize("scale_dtype", [torch.float32, torch.float16])
def test_int4_weight_quant_bit_exact(ops, scale_dtype):
    w = workloads.w4a4_linear(m=8, k=256, n=72, seed=3)["w"]
    q = torch.empty(72, 128, dtype=torch.uint8, device="cuda")
    s = torch.empty(72, 4, dtype=scale_dtype, device="cuda")
    ops.weight_quant_int4_g64(q, s, cu(w))
    p_ref, s_ref, _ = quant.int4_weight_quant_g64(w)
    assert_bit_equal(q, p_ref)
    assert_bit_equal(s, s_ref.to(scale_dtype))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_int8_weight_quant_bit_exact(ops, dtype):
    g = torch.Generator().manual_seed(9)
    w = (torch.randn(70, 650, generator=g) * 0.02).to(dtype)
    w[3] = 0
    pre = (0.25 + torch.rand(650, generator=g)).float()
    for p in (pre, None):
        qw = torch.empty(70, 650, dtype=torch.int8, device="cuda")
        sw = torch.empty(70, dtype=torch.float32, device="cuda")
        ops.invoke_get_int8_weight_scale(sw, qw, cu(w), cu(p))
        q_ref, s_ref = quant.int8_weight_quant_device(w, p)
        assert_bit_equal(sw, s_ref)
        assert_bit_equal(qw, q_ref)


def test_int8_weight_quant_against_reference_run_fixture(ops):
    """The device twin (lyraq_weight_quant_int8 = GetINT8WeightScale, quant_kernels.cu:173-223) beside the outputs of
    the reference's offline exporter function tensor_quant (tests/golden/ref_int8_weight_quant.npz, written by running
    that function).  The two rules differ by design: the device divides by s = amax/127 and saturates at -128, the
    exporter multiplies by 127/amax, clamps at -127 and returns scale 1 for amax <= 2**-24 where the device returns
    amax/127.  Stated bound on ordinary channels: at most one integer step on at most 0.1 % of the weights, scales
    reciprocal to 3e-7; zero channels give q = 0 in both."""
    import os
    import numpy as np
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_int8_weight_quant.npz"))
    for case in ("small_fp16", "k640_fp16"):           # weights the fixture holds as fp16 values: the device sees the same numbers
        w = torch.from_numpy(z[case + "_w"]).half()
        ref_q = torch.from_numpy(z[case + "_q"]).to(torch.int8)
        ref_scale = torch.from_numpy(z[case + "_scale"]).reshape(-1)
        n, k = w.shape
        qw = torch.empty(n, k, dtype=torch.int8, device="cuda")
        sw = torch.empty(n, dtype=torch.float32, device="cuda")
        ops.invoke_get_int8_weight_scale(sw, qw, cu(w), None)
        q, s = qw.cpu(), sw.cpu()
        amax = w.float().abs().amax(dim=1)
        ok = amax > 2.0 ** -14          # ordinary channels; the tiny ones are covered by the scale-1 rule stated above
        d = (q[ok].int() - ref_q[ok].int()).abs()
        assert int(d.max()) <= 1 and float((d != 0).float().mean()) <= 1e-3, case
        assert float((s[ok].double() * ref_scale[ok].double() - 1.0).abs().max()) < 3e-7
        if case == "small_fp16":
            assert int(q[3].abs().sum()) == 0


# Row statistics are summed in a different order on the device (fp32 shuffles) than in the oracle
# (fp64), so a value sitting on a rounding boundary may land one step away.  Stated tolerance:
# at most 1 LSB (int8) / 1 code (e4m3) / 1 ulp (16-bit y) on at most 0.1 % of the outputs.
def _close_y(got, want, frac=1e-3):
    """y = T(T(m * x_hat) + shift): a one-ulp step of x_hat moves y by about one ulp of the PRODUCT, which after
    cancellation against the shift can be several ulps of y itself, so the bound is absolute: 2 ulps of T at the
    magnitude of the terms (|m * x_hat| < 8 here), on at most `frac` of the outputs."""
    eps = 2.0 ** -8 if got.dtype == torch.bfloat16 else 2.0 ** -11
    g, w = got.cpu().float(), want.float()
    d = (g - w).abs()
    assert float(d.max()) <= 2 * eps * max(8.0, float(w.abs().max())), float(d.max())
    assert float((d != 0).float().mean()) <= frac


def _close(got, want, frac=1e-3):
    got = got.cpu()
    d = (got.to(torch.int32) - want.to(torch.int32)).abs()
    assert int(d.max()) <= 1, int(d.max())
    assert float((d != 0).float().mean()) <= frac


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,s,d", [(1, 37, 3072), (3, 11, 128), (2, 130, 1536), (8, 16, 3072)])
def test_adaln_quant_against_oracle(ops, dtype, b, s, d):
    a = workloads.adaln_input(b=b, s=s, d=d, seed=b * 100 + s, dtype=dtype)
    f8 = torch.tensor([0.02], dtype=torch.float32)
    ref = norms.adaln_quant(a["x"], a["scale"], a["shift"], fp8_scale=f8)
    y = torch.empty(b, s, d, dtype=dtype, device="cuda")
    q8 = torch.empty(b * s, d, dtype=torch.int8, device="cuda")
    s8 = torch.empty(b * s, dtype=torch.float32, device="cuda")
    qf8 = torch.empty(b * s, d, dtype=torch.uint8, device="cuda")
    ops.invoke_layer_norm_with_shift_and_scale(y, cu(a["x"]), cu(a["scale"]), cu(a["shift"]), 1e-6, q8=q8, q8_scale=s8,
                                               qf8=qf8, f8_scale=cu(f8))
    _close_y(y, ref["y"])
    # rows whose dynamic scale agrees bit for bit must agree on q8 up to the same slack
    same = (s8.cpu().view(torch.int32) == ref["s8"].view(torch.int32))
    assert float(same.float().mean()) >= 0.99
    _close(q8.cpu()[same], ref["q8"][same])
    # e4m3 codes: compare as sign-magnitude integers
    got = qf8.cpu().to(torch.int32)
    want = ref["qf8"].to(torch.int32)
    d_ = ((got & 0x7F) - (want & 0x7F)).abs()
    assert int(d_.max()) <= 1 and float((got != want).float().mean()) <= 1e-3
    # quantized-only call (no y) gives the same bytes
    q8b = torch.empty_like(q8)
    s8b = torch.empty_like(s8)
    ops.invoke_layer_norm_with_shift_and_scale(None, cu(a["x"]), cu(a["scale"]), cu(a["shift"]), 1e-6, q8=q8b, q8_scale=s8b)
    assert torch.equal(q8b, q8) and torch.equal(s8b, s8)


def test_adaln_two_e4m3_outputs_equal_two_single_passes(ops):
    w = workloads.adaln_input(b=2, s=70, d=3072, seed=9)
    sa, sb = torch.tensor([0.013]), torch.tensor([0.027])
    rows = 2 * 70
    qa = torch.empty(rows, 3072, dtype=torch.uint8, device="cuda")
    qb = torch.empty_like(qa)
    y = torch.empty(2, 70, 3072, dtype=torch.bfloat16, device="cuda")
    ops.adaln_quant_fp8x2(y, qa, cu(sa), qb, cu(sb), cu(w["x"]), cu(w["scale"]), cu(w["shift"]))
    ra, rb = torch.empty_like(qa), torch.empty_like(qa)
    y1 = torch.empty_like(y)
    ops.invoke_layer_norm_with_shift_and_scale(y1, cu(w["x"]), cu(w["scale"]), cu(w["shift"]), qf8=ra, f8_scale=cu(sa))
    ops.invoke_layer_norm_with_shift_and_scale(None, cu(w["x"]), cu(w["scale"]), cu(w["shift"]), qf8=rb, f8_scale=cu(sb))
    check_status()
    assert_bit_equal(qa, ra.cpu())
    assert_bit_equal(qb, rb.cpu())
    assert_bit_equal(y, y1.cpu())
    # and without the 16-bit output
    qa2, qb2 = torch.empty_like(qa), torch.empty_like(qa)
    ops.adaln_quant_fp8x2(None, qa2, cu(sa), qb2, cu(sb), cu(w["x"]), cu(w["scale"]), cu(w["shift"]))
    assert_bit_equal(qa2, ra.cpu())
    assert_bit_equal(qb2, rb.cpu())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,s", [(1, 1), (1, 7), (2, 37), (3, 8), (1, 4608 + 3)])
def test_adaln_3072_row_kernel_gives_the_general_kernel_bytes(ops, dtype, b, s):
    """Rows of 3072 with a quantized output take a kernel of their own (one warp per row).  It sums in the general row
    kernel's order, so every output form must be byte-identical to the general kernel's: y, the e4m3 codes of one or
    two scales, and the dynamically scaled int8 codes with their per-token scales.  Row counts cover a lone row, a
    block that is not full (8 rows per block) and the FLUX sequence plus a ragged tail; b > 1 covers the per-batch
    scale / shift rows."""
    from lyradiff_b200 import _lib

    a = workloads.adaln_input(b=b, s=s, d=3072, seed=500 + b * 10 + s, dtype=dtype)
    xd, sc, sh = cu(a["x"]), cu(a["scale"]), cu(a["shift"])
    fa, fb = cu(torch.tensor([0.017])), cu(torch.tensor([0.031]))
    rows = b * s

    def run():
        out = {}
        for form in ("y+e4m3", "e4m3", "y+e4m3x2", "e4m3x2", "y+s8+e4m3", "s8"):
            y = torch.full((b, s, 3072), float("nan"), dtype=dtype, device="cuda") if form.startswith("y") else None
            qa = torch.zeros(rows, 3072, dtype=torch.uint8, device="cuda")
            qb = torch.zeros_like(qa)
            q8 = torch.zeros(rows, 3072, dtype=torch.int8, device="cuda")
            s8 = torch.zeros(rows, dtype=torch.float32, device="cuda")
            if "x2" in form:
                ops.adaln_quant_fp8x2(y, qa, fa, qb, fb, xd, sc, sh)
            elif "s8" in form:
                if "e4m3" in form:
                    ops.invoke_layer_norm_with_shift_and_scale(y, xd, sc, sh, 1e-6, q8=q8, q8_scale=s8, qf8=qa, f8_scale=fa)
                else:
                    ops.invoke_layer_norm_with_shift_and_scale(y, xd, sc, sh, 1e-6, q8=q8, q8_scale=s8)
            else:
                ops.invoke_layer_norm_with_shift_and_scale(y, xd, sc, sh, 1e-6, qf8=qa, f8_scale=fa)
            check_status()
            out[form] = [t.cpu() for t in (y, qa, qb, q8, s8) if t is not None]
        return out

    L = _lib.lib()
    own = run()
    assert L.lyraq_debug_set_special_row_kernels(0) == 0
    try:
        general = run()
    finally:
        L.lyraq_debug_set_special_row_kernels(1)
    for form, tensors in own.items():
        for i, (t, g) in enumerate(zip(tensors, general[form])):
            assert t.dtype == g.dtype and torch.equal(t.view(torch.uint8), g.view(torch.uint8)), (form, i)


def test_adaln_golden(ops, golden):
    z = golden("adaln")
    b, s, d = z["x"].shape
    y = torch.empty(b, s, d, dtype=torch.bfloat16, device="cuda")
    q8 = torch.empty(b * s, d, dtype=torch.int8, device="cuda")
    s8 = torch.empty(b * s, dtype=torch.float32, device="cuda")
    qf8 = torch.empty(b * s, d, dtype=torch.uint8, device="cuda")
    ops.invoke_layer_norm_with_shift_and_scale(y, cu(z["x"]), cu(z["scale"]), cu(z["shift"]), 1e-6, q8=q8, q8_scale=s8,
                                               qf8=qf8, f8_scale=cu(z["f8_scale"]))
    _close_y(y, z["y"], frac=5e-3)
    _close(q8, z["q8"], frac=5e-3)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,dim", [(9, 64), (130, 320), (64, 640), (17, 1280), (5, 1024)])
def test_layernorm_int8_against_oracle(ops, dtype, rows, dim):
    g = torch.Generator().manual_seed(rows + dim)
    x = torch.randn(rows, dim, generator=g).to(dtype)
    res = torch.randn(rows, dim, generator=g).to(dtype)
    bias = (torch.randn(dim, generator=g) * 0.1).to(dtype)
    gamma = (1.0 + 0.1 * torch.randn(dim, generator=g)).to(dtype)
    beta = (0.1 * torch.randn(dim, generator=g)).to(dtype)
    pre = (0.5 + torch.rand(dim, generator=g)).float()
    s = torch.tensor([0.03], dtype=torch.float32)
    q = torch.empty(rows, dim, dtype=torch.int8, device="cuda")
    ops.invoke_layer_norm_int8o(q, cu(x), cu(gamma), cu(beta), cu(pre), cu(s), 1e-5)
    _close(q, norms.layernorm_int8(x, gamma, beta, pre, s)[0])
    hsum = torch.empty(rows, dim, dtype=dtype, device="cuda")
    ops.invoke_layer_norm_int8o(q, cu(x), cu(gamma), cu(beta), cu(pre), cu(s), 1e-5, residual=cu(res), bias=cu(bias),
                                sum_out=hsum)
    q_ref, h_ref = norms.layernorm_int8(x, gamma, beta, pre, s, residual=res, bias=bias)
    assert_bit_equal(hsum, h_ref, "x + residual + bias")
    _close(q, q_ref)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,dim", [(1, 320), (1, 640), (33, 640), (35, 320), (8192, 640), (4099, 320), (33, 1280), (2051, 1280)])
def test_layernorm_int8_short_row_kernel(ops, dtype, rows, dim):
    """Rows of 320, 640 and 1280 columns take a kernel in which 8, 16 or 32 lanes own a row (a warp works on 4, 2 or 1 rows
    at once).
    Its arithmetic is the general row kernel's except for the order of the two fp32 sums, so against the oracle it is
    held to the general kernel's tolerance, and against the general kernel itself to a tighter one; row counts that
    leave a warp's last rows empty are included."""
    from lyradiff_b200 import _lib

    g = torch.Generator().manual_seed(rows + dim)
    x = (torch.randn(rows, dim, generator=g) * 2.0 + 0.3).to(dtype)
    gamma = (1.0 + 0.1 * torch.randn(dim, generator=g)).to(dtype)
    beta = (0.1 * torch.randn(dim, generator=g)).to(dtype)
    pre = (0.5 + torch.rand(dim, generator=g)).float()
    s = torch.tensor([0.03], dtype=torch.float32)
    L = _lib.lib()
    for smooth in (pre, None):
        q = torch.full((rows, dim), 77, dtype=torch.int8, device="cuda")
        ops.invoke_layer_norm_int8o(q, cu(x), cu(gamma), cu(beta), cu(smooth), cu(s), 1e-5)
        check_status()
        if rows <= 64:
            _close(q, norms.layernorm_int8(x, gamma, beta, smooth, s)[0], frac=max(1e-3, 2.0 / (rows * dim)))
        assert L.lyraq_debug_set_special_row_kernels(0) == 0
        try:
            q_row = torch.full((rows, dim), 78, dtype=torch.int8, device="cuda")
            ops.invoke_layer_norm_int8o(q_row, cu(x), cu(gamma), cu(beta), cu(smooth), cu(s), 1e-5)
        finally:
            L.lyraq_debug_set_special_row_kernels(1)
        _close(q, q_row.cpu(), frac=max(1e-4, 2.0 / (rows * dim)))
    # the fused form: h = x + residual + bias is stored and normalised; the sum is element-wise, so it must be bit-equal
    res = (torch.randn(rows, dim, generator=g) * 0.5).to(dtype)
    bias = (torch.randn(dim, generator=g) * 0.1).to(dtype)
    for b in (bias, None):
        out = []
        for on in (1, 0):
            assert L.lyraq_debug_set_special_row_kernels(on) == 0
            try:
                q = torch.full((rows, dim), 79, dtype=torch.int8, device="cuda")
                hsum = torch.full((rows, dim), float("nan"), dtype=dtype, device="cuda")
                ops.invoke_layer_norm_int8o(q, cu(x), cu(gamma), cu(beta), cu(pre), cu(s), 1e-5, residual=cu(res), bias=cu(b),
                                            sum_out=hsum)
                check_status()
                out.append((q.cpu(), hsum.cpu()))
            finally:
                L.lyraq_debug_set_special_row_kernels(1)
        assert_bit_equal(out[0][1], out[1][1], "x + residual + bias")
        _close(out[0][0], out[1][0], frac=max(1e-4, 2.0 / (rows * dim)))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,dim", [(9, 64), (33, 1280), (8, 2560), (3, 5120)])
def test_geglu_int8_against_oracle(ops, dtype, rows, dim):
    g = torch.Generator().manual_seed(rows * 3 + dim)
    h = torch.randn(rows, 2 * dim, generator=g).to(dtype)
    b2 = (torch.randn(2 * dim, generator=g) * 0.1).to(dtype)
    pre = (0.5 + torch.rand(dim, generator=g)).float()
    s = torch.tensor([0.02], dtype=torch.float32)
    q = torch.empty(rows, dim, dtype=torch.int8, device="cuda")
    ops.invoke_fused_add_bias_geglu_int8o(q, cu(h), cu(b2), cu(pre), cu(s))
    # the device tanh is tanh.approx.f32 (as in the reference): 1 LSB on a small fraction
    _close(q, norms.geglu_int8(h, b2, pre, s), frac=2e-2)
    ops.invoke_fused_add_bias_geglu_int8o(q, cu(h), None, cu(pre), cu(s))
    _close(q, norms.geglu_int8(h, None, pre, s), frac=2e-2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,dim", [(1, 8), (9, 64), (33, 1288), (8192, 2560), (3, 16384)])
def test_geglu_flat_kernel_gives_the_row_kernel_bytes(ops, dtype, rows, dim):
    """Bias + GEGLU -> int8 has no row statistic and runs as a flat kernel over 8-column vectors; the general row kernel
    does the same arithmetic per vector, so the two must agree byte for byte: with and without the bias and the smoothing
    vector, from one vector to the SDXL feed-forward size (8192 x 2560), whose last block is partly idle, and the
    widest row."""
    from lyradiff_b200 import _lib

    g = torch.Generator().manual_seed(rows * 5 + dim)
    h = cu((torch.randn(rows, 2 * dim, generator=g) * 1.5).to(dtype))
    b2 = cu((torch.randn(2 * dim, generator=g) * 0.1).to(dtype))
    pre = cu((0.5 + torch.rand(dim, generator=g)).float())
    s = cu(torch.tensor([0.02], dtype=torch.float32))   # small enough that some codes saturate

    def run():
        out = []
        for bias, smooth in ((b2, pre), (None, pre), (b2, None), (None, None)):
            q = torch.zeros(rows, dim, dtype=torch.int8, device="cuda")
            ops.invoke_fused_add_bias_geglu_int8o(q, h, bias, smooth, s)
            check_status()
            out.append(q.cpu())
        return out

    L = _lib.lib()
    flat = run()
    assert L.lyraq_debug_set_special_row_kernels(0) == 0
    try:
        general = run()
    finally:
        L.lyraq_debug_set_special_row_kernels(1)
    for i, (a, b) in enumerate(zip(flat, general)):
        assert torch.equal(a, b), i
    assert int((flat[0] == 127).sum()) > 0 or rows * dim < 1000


def test_ln_geglu_golden(ops, golden):
    z = golden("ln_geglu")
    rows, dim = z["x"].shape
    q = torch.empty(rows, dim, dtype=torch.int8, device="cuda")
    ops.invoke_layer_norm_int8o(q, cu(z["x"]), cu(z["gamma"]), cu(z["beta"]), cu(z["pre"]), cu(z["scale"]), 1e-5)
    _close(q, z["q_ln"], frac=1e-2)
    ops.invoke_fused_add_bias_geglu_int8o(q, cu(z["h"]), cu(z["b2"]), cu(z["pre"]), cu(z["scale"]))
    _close(q, z["q_geglu"], frac=3e-2)


def test_adaln_full_size_properties(ops):
    """The FLUX AdaLN + quantize at full size ([4608, 3072]): dequantized int8 reproduces y within half a step per token,
    and the e4m3 output decodes to y within e4m3 spacing."""
    a = workloads.adaln_input(b=1, s=4608, d=3072, seed=0)
    xd, sc, sh = cu(a["x"]), cu(a["scale"]), cu(a["shift"])
    y = torch.empty(1, 4608, 3072, dtype=torch.bfloat16, device="cuda")
    q8 = torch.empty(4608, 3072, dtype=torch.int8, device="cuda")
    s8 = torch.empty(4608, dtype=torch.float32, device="cuda")
    qf8 = torch.empty(4608, 3072, dtype=torch.uint8, device="cuda")
    f8 = torch.tensor([8.0 / 448.0], dtype=torch.float32)
    ops.invoke_layer_norm_with_shift_and_scale(y, xd, sc, sh, 1e-6, q8=q8, q8_scale=s8, qf8=qf8, f8_scale=cu(f8))
    yf = y.view(4608, 3072).float()
    assert float((q8.float() * s8[:, None] - yf).abs().max() / s8.max()) <= 0.5 + 1e-3
    assert torch.equal(s8.cpu(), quant.dynamic_per_token_scale(y.view(4608, 3072).cpu(), None))
    dec = qf8.view(torch.float8_e4m3fn).float() * f8.cuda()
    assert float(((dec - yf).abs() / yf.abs().clamp_min(0.05)).max()) <= 0.0626 + 1e-3
    # oracle on a sample of rows
    rows = torch.arange(0, 4608, 97)
    ref = norms.adaln_quant(a["x"][:, rows], a["scale"], a["shift"], fp8_scale=f8)
    _close(q8.cpu()[rows], ref["q8"], frac=2e-3)
    check_status()


def test_nan_elements_and_subnormal_scales_take_the_exact_path(ops):
    """Inputs on which the division-free int8 / int4 rounding cannot be trusted: a NaN element (the reference's
    cvt.rni.sat gives 0 for it; a maximum taken with fmaxf ignores it) and a row / group whose scale is subnormal, so that
    1 / s is infinite.  Neither faults; both must give the oracle's bytes, i.e. the IEEE divide path."""
    g = torch.Generator().manual_seed(17)
    x = torch.randn(6, 256, generator=g).bfloat16()
    x[1, 5] = float("nan")
    x[2] = (torch.randn(256, generator=g) * 2.0 ** -131).bfloat16()        # amax / 127 and amax / 7 are subnormal
    x[3, 64:128] = (torch.randn(64, generator=g) * 2.0 ** -130).bfloat16()  # one subnormal-scale group in a normal row
    x[4, 200] = float("nan")
    x[4, 130:140] = 0.0
    # int8, dynamic per-token scales
    q = torch.empty(6, 256, dtype=torch.int8, device="cuda")
    sc = torch.empty(6, dtype=torch.float32, device="cuda")
    ops.invoke_sq_input_quant(q, cu(x), None, sc, dynamic=True)
    q_ref, s_ref = quant.sq_input_quant_dynamic(x, None)
    assert_bit_equal(sc, s_ref, "dynamic scales")
    assert_bit_equal(q, q_ref, "int8 with NaN / subnormal rows")
    assert int(q.cpu()[1, 5]) == 0 and int(q.cpu()[4, 200]) == 0
    # int4, groups of 64
    p4 = torch.empty(6, 128, dtype=torch.uint8, device="cuda")
    s4 = torch.empty(6, 4, dtype=torch.float32, device="cuda")
    ops.invoke_fused_quantize_and_lora_down_simple(None, p4, s4, cu(x), None, None)
    p_ref, s4_ref, _ = quant.int4_quant_g64(x, None)
    assert_bit_equal(s4, s4_ref, "int4 group scales")
    assert_bit_equal(p4, p_ref, "int4 with NaN / subnormal groups")
    check_status()
