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
