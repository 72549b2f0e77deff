"""GPU tests of the C++ torch custom classes (csrc/torch_classes.cpp): they issue the same launches as the Python mirrors in
lyradiff_b200.flux_blocks, which the oracle tests cover, so the outputs must agree bit for bit."""

import pytest
import torch

from tests.test_gpu_flux_block import _double_state_dict, _state_dict
from tests.util import check_status, cu

pytestmark = pytest.mark.gpu


def _rope(B, S, head_dim, g, dtype):
    ang = torch.rand(B, S, head_dim // 2, generator=g) * 6.28
    return torch.stack([torch.cos(ang), -torch.sin(ang), torch.sin(ang), torch.cos(ang)], dim=-1).reshape(
        B, S, head_dim // 2, 2, 2).to(dtype)


@pytest.fixture(scope="module")
def ns():
    from lyradiff_b200 import torch_classes
    return torch_classes.load()


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("level", [1, 2])
@pytest.mark.parametrize("B,S", [(1, 160), (2, 96), (2, 256)])
def test_single_block_same_bits_as_mirror(ns, dtype, level, B, S):
    from lyradiff_b200 import flux_blocks
    td = {"bf16": torch.bfloat16, "fp16": torch.float16}[dtype]
    D, heads, head_dim, mlp_scale = 256, 2, 128, 4
    g = torch.Generator().manual_seed(31 * level + S)
    prefix = "single_transformer_blocks.5."
    sd = _state_dict(prefix, D, mlp_scale, head_dim, level, g)
    hidden = cu(torch.randn(B, S, D, generator=g).to(td))
    temb = cu(torch.nn.functional.silu(torch.randn(B, D, generator=g)).to(td))
    rope = cu(_rope(B, S, head_dim, g, td))

    mirror = flux_blocks.FluxSingleTransformerBlockOp(dtype, D, heads, head_dim, mlp_scale, level)
    mirror.reload_model_from_state_dict(prefix, sd, "cuda")
    want = mirror.forward(hidden, rope, temb)

    op = ns.FluxSingleTransformerBlockOp(dtype, D, heads, head_dim, mlp_scale, level)
    op.initialize(ns.LyraDiffCommonContext())
    op.reload_model_from_state_dict(prefix, sd, "cuda")
    got = op.forward(hidden, rope, temb)
    check_status()
    assert got.dtype == td and tuple(got.shape) == (B, S, D)
    assert torch.equal(got, want)


@pytest.mark.parametrize("level", [1, 2])
@pytest.mark.parametrize("B,S,E", [(1, 128, 48), (2, 64, 24), (2, 256, 256)])
def test_double_block_same_bits_as_mirror(ns, level, B, S, E):
    from lyradiff_b200 import flux_blocks
    D, heads, head_dim = 256, 2, 128
    g = torch.Generator().manual_seed(17 * level + S)
    prefix = "transformer_blocks.1."
    sd = _double_state_dict(prefix, D, head_dim, level, g)
    hidden = cu(torch.randn(B, S, D, generator=g).bfloat16())
    encoder = cu(torch.randn(B, E, D, generator=g).bfloat16())
    temb = cu(torch.nn.functional.silu(torch.randn(B, D, generator=g)).bfloat16())
    rope = cu(_rope(B, E + S, head_dim, g, torch.bfloat16))

    mirror = flux_blocks.FluxTransformerBlockOp("bf16", D, heads, head_dim, 4, level)
    mirror.reload_model_from_state_dict(prefix, sd, "cuda")
    want_i, want_t = mirror.forward(hidden, encoder, rope, temb)

    op = ns.FluxTransformerBlockOp("bf16", D, heads, head_dim, 4, level)
    op.initialize(ns.LyraDiffCommonContext())
    op.reload_model_from_state_dict(prefix, sd, "cuda")
    got_i, got_t = op.forward(hidden, encoder, rope, temb)
    check_status()
    assert torch.equal(got_i, want_i) and torch.equal(got_t, want_t)


def test_forward_rejects_wrong_inputs(ns):
    g = torch.Generator().manual_seed(3)
    prefix = "b."
    op = ns.FluxSingleTransformerBlockOp("bf16", 256, 2, 128, 4, 1)
    op.reload_model_from_state_dict(prefix, _state_dict(prefix, 256, 4, 128, 1, g), "cuda")
    x = torch.zeros(1, 8, 256, dtype=torch.bfloat16, device="cuda")
    r = torch.zeros(1, 8, 64, 2, 2, dtype=torch.bfloat16, device="cuda")
    t = torch.zeros(1, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="inference dtype"):
        op.forward(x.half(), r, t)
    with pytest.raises(RuntimeError, match="shape mismatch"):
        op.forward(x, r[:, :4].contiguous(), t)
    with pytest.raises(RuntimeError, match="inference dtype"):
        op.forward(x.cpu(), r, t)


@pytest.mark.parametrize("level", [7, 8])
@pytest.mark.parametrize("B,S", [(1, 160), (2, 96)])
def test_single_block_int4_same_bits_as_mirror(ns, level, B, S):
    from lyradiff_b200 import flux_blocks
    from tests.test_gpu_flux_block import _int4_state_dict
    D, heads, head_dim, mlp_scale = 256, 2, 128, 4
    g = torch.Generator().manual_seed(13 * level + S)
    prefix = "single_transformer_blocks.2."
    sd = _int4_state_dict(prefix, D, mlp_scale, head_dim, level, g)
    hidden = cu(torch.randn(B, S, D, generator=g).bfloat16())
    temb = cu(torch.nn.functional.silu(torch.randn(B, D, generator=g)).bfloat16())
    rope = cu(_rope(B, S, head_dim, g, torch.bfloat16))

    mirror = flux_blocks.FluxSingleTransformerBlockOp("bf16", D, heads, head_dim, mlp_scale, level)
    mirror.reload_model_from_state_dict(prefix, sd, "cuda")
    want = mirror.forward(hidden, rope, temb)

    op = ns.FluxSingleTransformerBlockOp("bf16", D, heads, head_dim, mlp_scale, level)
    op.initialize(ns.LyraDiffCommonContext())
    op.reload_model_from_state_dict(prefix, sd, "cuda")
    got = op.forward(hidden, rope, temb)
    check_status()
    assert torch.equal(got, want)


@pytest.mark.parametrize("level", [7, 8])
def test_double_block_int4_same_bits_as_mirror(ns, level):
    from lyradiff_b200 import flux_blocks
    from tests.test_gpu_flux_block import _int4_double_state_dict
    D, heads, head_dim, B, S, E = 256, 2, 128, 2, 64, 24
    g = torch.Generator().manual_seed(19 * level)
    prefix = "transformer_blocks.0."
    sd = _int4_double_state_dict(prefix, D, head_dim, level, g)
    hidden = cu(torch.randn(B, S, D, generator=g).bfloat16())
    encoder = cu(torch.randn(B, E, D, generator=g).bfloat16())
    temb = cu(torch.nn.functional.silu(torch.randn(B, D, generator=g)).bfloat16())
    rope = cu(_rope(B, E + S, head_dim, g, torch.bfloat16))
    mirror = flux_blocks.FluxTransformerBlockOp("bf16", D, heads, head_dim, 6, level)
    mirror.reload_model_from_state_dict(prefix, sd, "cuda")
    want_i, want_t = mirror.forward(hidden, encoder, rope, temb)
    op = ns.FluxTransformerBlockOp("bf16", D, heads, head_dim, 6, level)
    op.initialize(ns.LyraDiffCommonContext())
    op.reload_model_from_state_dict(prefix, sd, "cuda")
    got_i, got_t = op.forward(hidden, encoder, rope, temb)
    check_status()
    assert torch.equal(got_i, want_i) and torch.equal(got_t, want_t)


def test_levels_that_are_not_built_raise(ns):
    with pytest.raises(RuntimeError, match="quant_level"):
        ns.FluxTransformerBlockOp("bf16", 256, 2, 128, 4, 5)


@pytest.mark.parametrize("level", [1, 2])
def test_lora_hot_swap_same_bits_as_mirror(ns, level):
    from lyradiff_b200 import flux_blocks
    D, heads, head_dim, mlp_scale = 256, 2, 128, 4
    g = torch.Generator().manual_seed(90 + level)
    prefix = "s."
    sd = _state_dict(prefix, D, mlp_scale, head_dim, level, g)
    hidden = cu(torch.randn(1, 96, D, generator=g).bfloat16())
    temb = cu(torch.nn.functional.silu(torch.randn(1, D, generator=g)).bfloat16())
    rope = cu(_rope(1, 96, head_dim, g, torch.bfloat16))
    mirror = flux_blocks.FluxSingleTransformerBlockOp("bf16", D, heads, head_dim, mlp_scale, level)
    mirror.reload_model_from_state_dict(prefix, sd, "cuda")
    op = ns.FluxSingleTransformerBlockOp("bf16", D, heads, head_dim, mlp_scale, level)
    op.reload_model_from_state_dict(prefix, sd, "cuda")
    base = op.forward(hidden, rope, temb).clone()
    for names, shape in ((["proj_out"], (D, 5 * D)), (["attn", "to_qkv"], (3 * D, D)), (["norm", "linear"], (3 * D, D))):
        lora = cu((torch.randn(shape, generator=g) * 0.01).bfloat16())
        mirror.load_lora_by_name(names, lora, 0.8)
        op.load_lora_by_name(names, lora, 0.8)
    got = op.forward(hidden, rope, temb)
    assert torch.equal(got, mirror.forward(hidden, rope, temb)) and not torch.equal(got, base)
    op.load_lora_by_name(["attn", "to_k"], cu(torch.zeros(4, 4).bfloat16()), 1.0)   # unknown path: reported and skipped
    op.clear_lora()
    assert torch.equal(op.forward(hidden, rope, temb), base)
    check_status()


@pytest.mark.parametrize("level,file_type", [(2, "fp32"), (7, "fp32")])
def test_reload_from_bin_same_bits_as_state_dict(ns, tmp_path, level, file_type):
    import numpy as np
    from tests.test_gpu_flux_block import _int4_state_dict, _write_bins
    D, heads, head_dim, mlp_scale = 256, 2, 128, 4
    g = torch.Generator().manual_seed(95 + level)
    prefix = "single_transformer_blocks.1."
    sd = _int4_state_dict(prefix, D, mlp_scale, head_dim, level, g) if level == 7 else _state_dict(prefix, D, mlp_scale, head_dim, level, g)
    base = str(tmp_path) + "/" + prefix
    _write_bins(base, sd, prefix, np.float32)
    hidden = cu(torch.randn(1, 64, D, generator=g).bfloat16())
    temb = cu(torch.nn.functional.silu(torch.randn(1, D, generator=g)).bfloat16())
    rope = cu(_rope(1, 64, head_dim, g, torch.bfloat16))
    a = ns.FluxSingleTransformerBlockOp("bf16", D, heads, head_dim, mlp_scale, level)
    a.reload_model_from_state_dict(prefix, sd, "cuda")
    b = ns.FluxSingleTransformerBlockOp("bf16", D, heads, head_dim, mlp_scale, level)
    b.reload_model_from_bin(base, file_type)
    assert torch.equal(a.forward(hidden, rope, temb), b.forward(hidden, rope, temb))


def test_double_block_reload_from_bin_and_lora(ns, tmp_path):
    import numpy as np
    from tests.test_gpu_flux_block import _write_bins
    D, heads, head_dim = 256, 2, 128
    g = torch.Generator().manual_seed(99)
    prefix = "transformer_blocks.6."
    sd = _double_state_dict(prefix, D, head_dim, 1, g)
    base = str(tmp_path) + "/" + prefix
    _write_bins(base, sd, prefix, np.float16)
    sd16 = {k: (v.half() if v.dtype == torch.bfloat16 else v) for k, v in sd.items()}
    hidden = cu(torch.randn(1, 64, D, generator=g).half())
    encoder = cu(torch.randn(1, 32, D, generator=g).half())
    temb = cu(torch.nn.functional.silu(torch.randn(1, D, generator=g)).half())
    rope = cu(_rope(1, 96, head_dim, g, torch.float16))
    a = ns.FluxTransformerBlockOp("fp16", D, heads, head_dim, 6, 1)
    a.reload_model_from_state_dict(prefix, sd16, "cuda")
    b = ns.FluxTransformerBlockOp("fp16", D, heads, head_dim, 6, 1)
    b.reload_model_from_bin(base, "fp16")
    want = a.forward(hidden, encoder, rope, temb)
    for u, v in zip(want, b.forward(hidden, encoder, rope, temb)):
        assert torch.equal(u, v)
    b.load_lora_by_name(["ff_context", "net.2"], cu((torch.randn(D, 4 * D, generator=g) * 0.02).half()), 1.0)
    out_i, out_t = b.forward(hidden, encoder, rope, temb)
    assert torch.equal(out_i, want[0]) and not torch.equal(out_t, want[1])   # only the text stream's FF changed
    b.clear_lora()
    for u, v in zip(want, b.forward(hidden, encoder, rope, temb)):
        assert torch.equal(u, v)


def test_densely_launched_forwards_repeat_bit_for_bit(ns):
    """The C++ class issues a block's launches back to back, so consecutive kernels overlap through dependent launch and
    run beside one another on the SMs, which the Python mirror's launch gaps never produce.  Sixty forwards in a row,
    with unrelated work in between to vary the timing, must give one and the same result (this is the test that caught
    an attention epilogue reading its accumulator one product early)."""
    from lyradiff_b200 import flux_blocks
    D, heads, head_dim, B, S, E, level = 256, 2, 128, 2, 256, 256, 2
    g = torch.Generator().manual_seed(91)
    prefix = "transformer_blocks.0."
    sd = _double_state_dict(prefix, D, head_dim, level, g)
    hidden = cu(torch.randn(B, S, D, generator=g).bfloat16())
    encoder = cu(torch.randn(B, E, D, generator=g).bfloat16())
    temb = cu(torch.nn.functional.silu(torch.randn(B, D, generator=g)).bfloat16())
    rope = cu(_rope(B, E + S, head_dim, g, torch.bfloat16))
    mirror = flux_blocks.FluxTransformerBlockOp("bf16", D, heads, head_dim, 4, level)
    mirror.reload_model_from_state_dict(prefix, sd, "cuda")
    want_i, want_t = (t.clone() for t in mirror.forward(hidden, encoder, rope, temb))
    op = ns.FluxTransformerBlockOp("bf16", D, heads, head_dim, 4, level)
    op.initialize(ns.LyraDiffCommonContext())
    op.reload_model_from_state_dict(prefix, sd, "cuda")
    junk = torch.randn(2048, 2048, device="cuda")
    bad = 0
    for it in range(60):
        if it % 3 == 0:
            junk = torch.tanh(junk @ junk * 1e-3)
        got_i, got_t = op.forward(hidden, encoder, rope, temb)
        bad += int(not (torch.equal(got_i, want_i) and torch.equal(got_t, want_t)))
    check_status()
    assert bad == 0, "%d of 60 forwards differ" % bad
