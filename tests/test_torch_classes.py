"""The C++ torch custom classes load without a GPU, carry the reference's class and method names
(src/lyradiff/th_op/pybind.cc:9-96) and refuse what is not built the way the Python mirrors do."""

import pytest
import torch

METHODS = ["initialize", "forward", "reload_model_from_state_dict", "reload_model_from_bin", "load_lora_by_name", "clear_lora"]


@pytest.fixture(scope="module")
def ns():
    from lyradiff_b200 import build, torch_classes
    build.build_classes()
    return torch_classes.load()


@pytest.mark.parametrize("name", ["FluxSingleTransformerBlockOp", "FluxTransformerBlockOp"])
def test_names_and_signatures(ns, name):
    cls = getattr(ns, name)
    op = cls("bf16", 256, 2, 128, 4, 1)
    op.initialize(ns.LyraDiffCommonContext())
    for m in METHODS:
        assert callable(getattr(op, m)), m
    with pytest.raises(RuntimeError, match="quant_level"):
        cls("bf16", 256, 2, 128, 4, 0)
    with pytest.raises(RuntimeError, match="inference_dtype"):
        cls("fp32", 256, 2, 128, 4, 1)
    with pytest.raises(RuntimeError, match="embedding_dim"):
        cls("fp16", 256, 3, 128, 4, 1)
    with pytest.raises(RuntimeError, match="wrong model_dtype"):
        op.reload_model_from_bin("/nowhere/", "bf16")          # file types are fp32 and fp16, as in the reference
    with pytest.raises(RuntimeError, match="weight file missing"):
        op.reload_model_from_bin("/nowhere/", "fp16")
    with pytest.raises(RuntimeError, match="weights not loaded"):
        op.load_lora_by_name(["a"], torch.zeros(1), 1.0)
    with pytest.raises(RuntimeError, match="weights not loaded"):
        op.clear_lora()


def test_forward_needs_weights(ns):
    op = ns.FluxSingleTransformerBlockOp("bf16", 256, 2, 128, 4, 1)
    with pytest.raises(RuntimeError, match="weights not loaded"):
        op.forward(torch.zeros(1, 8, 256), torch.zeros(1, 8, 64, 2, 2), torch.zeros(1, 256))
    op2 = ns.FluxTransformerBlockOp("bf16", 256, 2, 128, 4, 2)
    with pytest.raises(RuntimeError, match="weights not loaded"):
        op2.forward(torch.zeros(1, 8, 256), torch.zeros(1, 4, 256), torch.zeros(1, 12, 64, 2, 2), torch.zeros(1, 256))


def test_missing_state_dict_key_raises(ns):
    op = ns.FluxSingleTransformerBlockOp("bf16", 256, 2, 128, 4, 1)
    with pytest.raises((RuntimeError, IndexError, KeyError)):
        op.reload_model_from_state_dict("p.", {"p.attn.to_qkv.weight": torch.zeros(768, 256)}, "cpu")


def test_whole_model_class_is_registered_with_the_reference_defaults(ns):
    op = ns.FluxTransformer2DModelOp("bf16", 16, 1, 1, 128, 2, 32, 64, True, 1)
    op.initialize(ns.LyraDiffCommonContext())
    for m in ("transformer_forward", "reload_transformer_model", "reload_transformer_model_from_state_dict", "load_lora_by_name",
              "clear_lora"):
        assert callable(getattr(op, m)), m
    with pytest.raises(RuntimeError, match="weights not loaded"):
        op.clear_lora()
    with pytest.raises(RuntimeError, match="wrong model_dtype"):
        op.reload_transformer_model("/nowhere", "bf16")
    with pytest.raises(RuntimeError, match="weight file missing"):
        op.reload_transformer_model("/nowhere", "fp32")
    with pytest.raises(RuntimeError, match="guidance"):
        ns.FluxTransformer2DModelOp("bf16", 16, 1, 1, 128, 2, 32, 64, False, 1)
    # keyword construction with the defaults of th_op/pybind.cc:13-27 (quant_level 0 is not built here)
    with pytest.raises(RuntimeError, match="quant_level"):
        ns.FluxTransformer2DModelOp(num_layers=1, num_single_layers=1)


def test_block_classes_take_the_reference_keywords_and_defaults(ns):
    """th_op/pybind.cc:66-96: inference_dtype="bf16", embedding_dim=3072, embedding_head_num=24, embedding_head_dim=128,
    mlp_scale=6 (double-stream) / 4 (single-stream), quant_level=0.  Level 0 is not built here, so the all-default
    construction is refused by name; with a built level the keywords and the other defaults go through."""
    for cls in (ns.FluxSingleTransformerBlockOp, ns.FluxTransformerBlockOp):
        with pytest.raises(RuntimeError, match="quant_level 0"):
            cls()
        op = cls(quant_level=1)                                   # every other argument at its default
        with pytest.raises(RuntimeError, match="weights not loaded"):
            op.clear_lora()
        op = cls(inference_dtype="fp16", embedding_dim=256, embedding_head_num=2, embedding_head_dim=128, quant_level=2)
        with pytest.raises(RuntimeError, match="embedding_dim must equal"):
            cls(embedding_dim=512, embedding_head_num=2, embedding_head_dim=128, quant_level=1)
