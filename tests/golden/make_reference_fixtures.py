"""Writes tests/golden/ref_*.npz: outputs of the REFERENCE's own Python functions on seeded inputs.

    python tests/golden/make_reference_fixtures.py path/to/lyraDiff-checkout

Three functions of the reference are plain torch and run on a CPU once they are lifted out of their modules (the
modules themselves import diffusers / modelopt, which are not installed, so the function definitions are taken from the
parsed source by name and executed unchanged in a namespace that holds only torch):

* tensor_quant   lyradiff/convert_model_scripts/convert_sd_quant_model.py:108-155 - the offline INT8 weight rule
* to_float8      lyradiff/convert_model_scripts/convert_flux_fp8_safetensors.py:9-22 - the offline e4m3 weight cast
* rope, EmbedND  lyradiff/lyradiff_model/lyradiff_flux_transformer_model_v2.py:35-65 - the rotary table the block ops get

The fixtures hold the inputs and what the reference returned; tests compare the CPU oracle (and the library's host
code) with them, so the checkout is needed only to regenerate the files, never to run the tests.
"""

import ast
import contextlib
import io
import os
import sys
from typing import List

import numpy as np
import torch
from torch import nn

HERE = os.path.dirname(os.path.abspath(__file__))


def lift(path, names):
    """Returns {name: object} for the top-level functions/classes `names` of the python file at `path`."""
    with open(path, "r", encoding="utf8") as f:
        tree = ast.parse(f.read())
    picked = [n for n in tree.body if isinstance(n, (ast.FunctionDef, ast.ClassDef)) and n.name in names]
    assert sorted(n.name for n in picked) == sorted(names), (path, [n.name for n in picked])
    ns = {"torch": torch, "nn": nn, "List": List}
    exec(compile(ast.Module(body=picked, type_ignores=[]), path, "exec"), ns)
    return {n: ns[n] for n in names}


def int8_weight_cases(g):
    """Weight matrices [N, K] for the per-output-channel rule, with the corner rows the rule special-cases."""
    w = torch.randn(40, 64, generator=g) * 0.02
    w[3] = 0.0                                   # all-zero channel: amax = 0
    w[5] = torch.randn(64, generator=g) * 2.0 ** -27   # amax below 2**-24
    w[7, :] = 0.0
    w[7, 11] = 2.0 ** -24                        # amax exactly at the threshold
    w[9] = torch.linspace(-1.0, 1.0, 64)         # hits +-127 and exact .5 ties after scaling
    w[11, 0] = 3.0                               # one large outlier
    big = torch.randn(24, 640, generator=g) * 0.02
    return {"small": w, "k640": big, "small_fp16": w.half(), "k640_fp16": big.half()}


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_reference_fixtures.py <checkout of the reference repository>")
    ref = sys.argv[1]
    g = torch.Generator().manual_seed(20240607)

    # ---- tensor_quant: INT8 weights, per output channel (amax [N, 1] as the exporter passes it, :209-219)
    tq = lift(os.path.join(ref, "lyradiff/convert_model_scripts/convert_sd_quant_model.py"), ["tensor_quant"])["tensor_quant"]
    out = {}
    for name, w in int8_weight_cases(g).items():
        amax = w.float().abs().amax(dim=1, keepdim=True)
        q, scale = tq(w.clone(), amax.clone())
        out[name + "_w"] = w.float().numpy()
        out[name + "_is_half"] = np.array(w.dtype == torch.half)
        out[name + "_amax"] = amax.numpy()
        out[name + "_q"] = q.float().numpy()
        out[name + "_scale"] = scale.float().numpy()
    np.savez_compressed(os.path.join(HERE, "ref_int8_weight_quant.npz"), **out)

    # ---- to_float8: e4m3 weight cast with a given amax (prints finfo.max; silenced)
    f8 = lift(os.path.join(ref, "lyradiff/convert_model_scripts/convert_flux_fp8_safetensors.py"), ["to_float8"])["to_float8"]
    x = torch.randn(48, 96, generator=g) * 0.02
    x[0, :8] = torch.tensor([0.0, -0.0, 1e-9, -1e-9, 0.08, -0.08, 0.0801, 0.5])   # zeros, underflow, the amax itself, beyond it
    out = {}
    for name, amax in (("own_amax", x.abs().max()), ("tight_amax", torch.tensor(0.05))):
        with contextlib.redirect_stdout(io.StringIO()):
            q, inv = f8(x.clone(), amax.clone())
        out[name + "_amax"] = amax.reshape(1).numpy()
        out[name + "_codes"] = q.view(torch.uint8).numpy()
        out[name + "_inv_scale"] = inv.reshape(1).numpy()
    out["x"] = x.numpy()
    np.savez_compressed(os.path.join(HERE, "ref_fp8_weight_cast.npz"), **out)

    # ---- rope / EmbedND: FLUX position ids -> [B, 1, S, 64, 2, 2] table (axes 16 + 56 + 56, theta 10000)
    fx = lift(os.path.join(ref, "lyradiff/lyradiff_model/lyradiff_flux_transformer_model_v2.py"), ["rope", "EmbedND"])
    txt, hh, ww = 5, 4, 6
    ids = torch.zeros(1, txt + hh * ww, 3)
    ids[0, txt:, 1] = torch.arange(hh).repeat_interleave(ww).float()
    ids[0, txt:, 2] = torch.arange(ww).repeat(hh).float()
    emb = fx["EmbedND"](128, 10000, [16, 56, 56])(ids)
    one_axis = fx["rope"](torch.tensor([[0.0, 1.0, 2.0, 63.0, 127.0]]), 16, 10000)
    np.savez_compressed(os.path.join(HERE, "ref_rope_table.npz"), ids=ids.numpy(), table=emb.numpy(),
                        axes_dim=np.array([16, 56, 56]), theta=np.array(10000), one_axis_pos=np.array([0.0, 1.0, 2.0, 63.0, 127.0]),
                        one_axis_table=one_axis.numpy())
    print("wrote ref_int8_weight_quant.npz ref_fp8_weight_cast.npz ref_rope_table.npz")


if __name__ == "__main__":
    main()
