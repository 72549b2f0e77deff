"""Loader of the C++ torch custom classes `torch.classes.lyradiff.*` (csrc/torch_classes.cpp), the form in which the
reference exposes its blocks to Python (src/lyradiff/th_op/pybind.cc:9-96; its users call
`torch.classes.load_library(<path of the built .so>)` and then `torch.classes.lyradiff.FluxSingleTransformerBlockOp(...)`).

    from lyradiff_b200 import torch_classes
    ns = torch_classes.load()                                   # == torch.classes.lyradiff
    op = ns.FluxSingleTransformerBlockOp("bf16", 3072, 24, 128, 4, 1)
    op.initialize(ns.LyraDiffCommonContext())
    op.reload_model_from_state_dict(prefix, state_dict, "cuda")
    out = op.forward(hidden_states, rope_emb, temb)

The classes run the same launches as the Python mirrors in flux_blocks.py and give the same bits.  The library must have
been built (python -m lyradiff_b200.build); a missing file raises, nothing falls back.
"""

import os

import torch

LIB = os.path.join(os.path.dirname(os.path.abspath(__file__)), "liblyradiff_classes.so")
_loaded = False


def load():
    global _loaded
    if not _loaded:
        if not os.path.exists(LIB):
            raise RuntimeError("%s is not built: run `python -m lyradiff_b200.build`" % LIB)
        torch.classes.load_library(LIB)
        _loaded = True
    return torch.classes.lyradiff
