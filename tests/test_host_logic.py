"""Host-side logic of the block / model mirrors that needs no GPU: LoRA name routing, the .bin manifests and reader, and the
meaning of the loaders' `device` argument."""

import warnings

import numpy as np
import pytest
import torch

from lyradiff_b200 import flux_blocks, flux_model


class _Target:
    def __init__(self):
        self.loaded, self.cleared = [], 0

    def load_lora(self, weight, scale):
        self.loaded.append((tuple(weight.shape), scale))

    def clear_lora(self):
        self.cleared += 1


def test_lora_names_walk_the_nested_table_and_unknown_paths_are_reported():
    a, b, c = _Target(), _Target(), _Target()
    table = {"attn": {"to_qkv": a, "to_out.0": b}, "proj_mlp": c}
    flux_blocks._load_lora_by_name(table, ["attn", "to_out.0"], torch.zeros(2, 3), 0.5)
    flux_blocks._load_lora_by_name(table, ["proj_mlp"], torch.zeros(4, 1), 1.0)
    assert b.loaded == [((2, 3), 0.5)] and c.loaded == [((4, 1), 1.0)] and a.loaded == []
    for bad in (["attn"], ["attn", "to_k"], ["nothing"], ["proj_mlp", "deeper"]):
        with pytest.warns(UserWarning, match="cannot find"):
            flux_blocks._load_lora_by_name(table, bad, torch.zeros(1), 1.0)
    flux_blocks._clear_lora(table)
    assert (a.cleared, b.cleared, c.cleared) == (1, 1, 1)


@pytest.mark.parametrize("level,count", [(1, 13), (2, 14), (7, 27), (8, 28)])
def test_single_block_bin_manifest(level, count):
    op = flux_blocks.FluxSingleTransformerBlockOp("bf16", 3072, 24, 128, 4, level)
    files = op._bin_files()
    assert len(files) == count and len({k for k, _, _ in files}) == count
    shapes = {k: s for k, s, _ in files}
    assert shapes["norm.linear.weight"] == (9216, 3072) and shapes["attn.norm_q.weight"] == (128,)
    if level in (7, 8):
        assert shapes["proj_out.linears.1.linear.packed_weight"] == (3072, 6144) and "proj_out.linears.1.linear.bias" not in shapes
        assert shapes["attn.to_qkv.weight_scale"] == (9216, 48) and shapes["proj_mlp.lora_down"] == (32, 3072)
    else:
        assert shapes["proj_out.weight"] == (3072, 15360) and shapes["proj_mlp_input_scale"] == (1,)
    assert ("norm.linear_input_scale" in shapes) == (level in (2, 8))


def test_model_manifest_prefixes_every_block():
    op = flux_model.FluxTransformer2DModelOp("bf16", 64, 2, 3, 128, 24, 768, 4096, True, 1)
    keys = [k for k, _, _ in op._bin_files()]
    assert len(keys) == len(set(keys))
    assert "transformer_blocks.1.ff_context.net.2_input_scale" in keys and "single_transformer_blocks.2.proj_out.bias" in keys
    assert "time_text_embed.text_embedder.linear_1.weight" in keys and "norm_out.linear.bias" in keys
    assert dict((k, s) for k, s, _ in op._bin_files())["time_text_embed.text_embedder.linear_1.weight"] == (3072, 768)


def test_bin_reader_types_sizes_and_missing_files(tmp_path):
    base = str(tmp_path) + "/blk."
    np.arange(6, dtype=np.float16).tofile(base + "w.bin")
    np.array([0.25], dtype=np.float32).tofile(base + "s.bin")
    np.arange(-4, 4, dtype=np.int8).tofile(base + "p.bin")
    sd = flux_blocks._state_dict_from_bin(base, "fp16", [("w", (2, 3), "T"), ("s", (1,), "f32"), ("p", (2, 4), "i8")])
    assert sd["w"].dtype == torch.float16 and sd["w"].tolist() == [[0, 1, 2], [3, 4, 5]]
    assert sd["s"].dtype == torch.float32 and float(sd["s"]) == 0.25
    assert sd["p"].dtype == torch.int8 and sd["p"][0].tolist() == [-4, -3, -2, -1]
    with pytest.raises(RuntimeError, match="missing or too small"):
        flux_blocks._state_dict_from_bin(base, "fp32", [("w", (2, 3), "T")])       # 12 bytes on disk, 24 wanted
    with pytest.raises(RuntimeError, match="missing or too small"):
        flux_blocks._state_dict_from_bin(base, "fp16", [("absent", (1,), "T")])
    with pytest.raises(ValueError, match="wrong model_dtype"):
        flux_blocks._state_dict_from_bin(base, "bf16", [("w", (2, 3), "T")])


def test_device_argument_is_validated_before_anything_is_loaded():
    op = flux_blocks.FluxSingleTransformerBlockOp("bf16", 256, 2, 128, 4, 1)
    with pytest.raises(RuntimeError, match="where the state dict"):
        op.reload_model_from_state_dict("p.", {}, "tpu")
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        with pytest.raises(RuntimeError, match="weights not loaded"):
            op.clear_lora()


def test_sdxl_int8_bin_manifest_names_the_reference_files():
    from lyradiff_b200 import layers
    files = layers.SmoothQuantLinear.bin_files("attn1.to_qkv", 1920, 640, has_bias=False)
    assert [f[0] for f in files] == ["attn1.to_qkv.weight_int8.bin", "attn1.to_qkv.weight_quant_scale.bin",
                                     "attn1.to_qkv.input_quant_scale.bin", "attn1.to_qkv.pre_quant_scale.bin"]
    assert [f[2] for f in files] == [(1920, 640), (1920,), (1,), (640,)]
    assert layers.SmoothQuantLinear.bin_files("ff.net.2", 640, 2560)[-1] == ("ff.net.2.bias.bin", "model", (640,))


def test_unbuilt_quant_levels_are_refused_by_name():
    """The reference's constructors default to quant_level 0 (16-bit); this library builds the quantized levels only and
    says so at construction, in the mirrors as in the C++ classes."""
    for level in (0, 3, 5):
        with pytest.raises(NotImplementedError, match="only 1, 2"):
            flux_blocks.FluxSingleTransformerBlockOp("bf16", 3072, 24, 128, 4, level)
        with pytest.raises(NotImplementedError, match="only 1, 2"):
            flux_blocks.FluxTransformerBlockOp("bf16", 3072, 24, 128, 6, level)
    with pytest.raises(NotImplementedError):
        flux_blocks.FluxSingleTransformerBlockOp()            # the reference's default arguments


def test_bench_reference_arm_prints_exactly_one_json_line(tmp_path):
    """What reads bench.py's output takes its standard output as one JSON line: nothing else may be written there (progress
    and libraries' banners go to standard error).  The reference arm runs on the host cores, so this needs no GPU."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--case", "adaln_quant", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=300, cwd=root)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = r.stdout.splitlines()
    assert len(lines) == 1, lines
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["n_gpus"] == 1 and line["steps"] == 1
    for key in ("metric", "value", "unit", "ms_per_step", "higher_is_better", "config", "e2e", "cpu_baseline"):
        assert key in line, key
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
