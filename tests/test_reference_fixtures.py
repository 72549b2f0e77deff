"""The CPU oracle and the library's host code against outputs of the reference's OWN Python functions.

tests/golden/ref_*.npz were written by tests/golden/make_reference_fixtures.py, which executes three plain-torch
functions of the reference unchanged (tensor_quant, to_float8, rope / EmbedND).  These are the only pieces of the
reference that run without a GPU, so they are what pins the oracle to something the reference computed.
"""

import os

import numpy as np
import torch

from oracle import e4m3, norms, quant

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    return np.load(os.path.join(GOLD, name))


# ------------------------------------------------------------------ INT8 weight rule (offline exporter)
def test_int8_weight_quant_offline_equals_reference_tensor_quant():
    z = _load("ref_int8_weight_quant.npz")
    for case in ("small", "k640", "small_fp16", "k640_fp16"):
        w = torch.from_numpy(z[case + "_w"])
        if bool(z[case + "_is_half"]):
            w = w.half()
        q, s = quant.int8_weight_quant_offline(w)
        ref_q = torch.from_numpy(z[case + "_q"]).to(torch.int8)
        ref_scale = torch.from_numpy(z[case + "_scale"]).reshape(-1)       # the reference returns 127/amax (1 where amax ~ 0)
        assert torch.equal(q, ref_q), case
        amax = torch.from_numpy(z[case + "_amax"]).reshape(-1)
        tiny = amax <= 2.0 ** -24
        # the exporter stores 1/scale per channel (convert_sd_quant_model.py:209-219): for tiny channels both are 1
        assert torch.equal(s[tiny], torch.ones(int(tiny.sum())))
        assert torch.equal(ref_scale[tiny], torch.ones(int(tiny.sum())))
        # elsewhere s_w = amax/127 and the reference's 127/amax are reciprocals up to fp32 rounding
        prod = (s[~tiny].double() * ref_scale[~tiny].double())
        assert float((prod - 1.0).abs().max()) < 3e-7, case
        # corner rows of the fixture: zero channel, sub-threshold channel, threshold channel -> all zeros
        if case.startswith("small"):
            assert int(q[3].abs().sum()) == 0 and int(q[5].abs().sum()) == 0 and int(q[7].abs().sum()) == 0
            assert int(q[9].max()) == 127 and int(q[9].min()) == -127       # narrow range: never -128


def test_int8_device_twin_differs_from_offline_rule_only_where_stated():
    """GetINT8WeightScale (quant_kernels.cu:173-223) divides by amax/127 and saturates to -128; the offline rule
    multiplies by 127/amax and clamps to -127.  On ordinary rows they agree except for ties broken by the two
    roundings; on a zero row the device twin returns scale 0 and the offline rule scale 1 (both q = 0)."""
    z = _load("ref_int8_weight_quant.npz")
    w = torch.from_numpy(z["k640_w"])
    q_off, s_off = quant.int8_weight_quant_offline(w)
    q_dev, s_dev = quant.int8_weight_quant_device(w, None)
    assert float((q_off != q_dev).float().mean()) < 1e-3
    assert int((q_off.int() - q_dev.int()).abs().max()) <= 1
    assert float(((s_off - s_dev).abs() / s_off).max()) < 2e-7
    w0 = torch.from_numpy(z["small_w"])
    q0, s0 = quant.int8_weight_quant_device(w0, None)
    assert int(q0[3].abs().sum()) == 0 and float(s0[3]) == 0.0
    assert float(quant.int8_weight_quant_offline(w0)[1][3]) == 1.0


# ------------------------------------------------------------------ e4m3 weight cast (offline exporter)
def test_e4m3_encode_equals_reference_to_float8():
    z = _load("ref_fp8_weight_cast.npz")
    x = torch.from_numpy(z["x"])
    for case in ("own_amax", "tight_amax"):
        amax = torch.from_numpy(z[case + "_amax"])[0]
        ref_codes = z[case + "_codes"]
        # the reference multiplies by 448/amax and clamps to +-448 before torch's cast: same arithmetic, then the oracle's encoder
        fwd = torch.tensor(448.0) / amax
        got = quant.fp8_quant(x, fwd.reshape(1), invert_scale=False).numpy()
        # the only representation difference: torch keeps the sign of -0.0 and of negative underflow, as the encoder does
        assert np.array_equal(got, ref_codes), (case, int((got != ref_codes).sum()))
        # the device path multiplies by fl(1/s) with s = amax/448 (memory_utils.cu:431-439): at most one code away, rarely
        s = (amax / torch.tensor(448.0)).reshape(1)
        dev = quant.fp8_quant(x, s, invert_scale=True).numpy()
        differs = dev != ref_codes
        assert differs.mean() < 5e-3, case
        step = np.abs(dev.astype(np.int16) - ref_codes.astype(np.int16))
        assert step.max() <= 1
        inv = torch.from_numpy(z[case + "_inv_scale"])[0]
        assert abs(float(inv) / float(s[0]) - 1.0) < 3e-7
    assert e4m3.decode(_load("ref_fp8_weight_cast.npz")["tight_amax_codes"]).max() == 448.0     # saturated, not NaN


# ------------------------------------------------------------------ rotary table
def test_rope_table_layout_and_values_equal_reference():
    from lyradiff_b200 import rope
    z = _load("ref_rope_table.npz")
    ids = torch.from_numpy(z["ids"])
    ref = torch.from_numpy(z["table"])
    got = rope.flux_rope_table(ids, tuple(int(a) for a in z["axes_dim"]), int(z["theta"]))
    assert got.shape == ref.shape == (1, 1, ids.shape[1], 64, 2, 2) and got.dtype == torch.float32
    # float64 cos/sin rounded to fp32: libm differences between hosts stay far below half an fp32 ulp of 1
    assert float((got - ref).abs().max()) <= 6e-8
    one = rope.axis_table(torch.from_numpy(z["one_axis_pos"]).reshape(1, -1), 16, 10000)
    assert float((one - torch.from_numpy(z["one_axis_table"])).abs().max()) <= 6e-8
    assert torch.equal(rope.flux_position_ids(5, 4, 6), ids)
    # layout: [.., i, 0, 0] = cos, [.., i, 0, 1] = -sin, [.., i, 1, 0] = sin, [.., i, 1, 1] = cos
    assert torch.equal(ref[..., 0, 0], ref[..., 1, 1]) and torch.equal(ref[..., 0, 1], -ref[..., 1, 0])
    assert torch.equal(ref[0, 0, :5], torch.eye(2).expand(5, 64, 2, 2))          # text rows: position 0 -> identity


def test_oracle_rmsnorm_rope_rotates_with_the_reference_table():
    """oracle.norms.rmsnorm_rope consumes the reference's table layout: with unit norm weights, a head rotated by the
    fixture's table equals complex multiplication by cos + i sin of the same angles."""
    z = _load("ref_rope_table.npz")
    table = torch.from_numpy(z["table"])[0, 0]                     # [S, 64, 2, 2]
    S = table.shape[0]
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(S, 3 * 128, generator=g)
    out = norms.rmsnorm_rope(qkv, torch.ones(256), table, 1, 128, eps=1e-6).reshape(S, 3, 128)
    x = qkv.reshape(S, 3, 128)[:, :2]
    xn = x / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-6).float()
    zc = torch.complex(xn[..., 0::2], xn[..., 1::2]) * torch.complex(table[:, None, :, 0, 0], table[:, None, :, 1, 0])
    want = torch.stack([zc.real, zc.imag], dim=-1).reshape(S, 2, 128)
    assert float((out[:, :2] - want).abs().max()) < 1e-5
    assert torch.equal(out[:, 2], qkv.reshape(S, 3, 128)[:, 2])
