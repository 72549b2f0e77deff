"""lyraq: lyraDiff's quantized-linear path for B200 (sm_100a).

    _lib          the C-ABI library liblyraq.so (ctypes; raises when it is not built -- there is no fallback)
    ops           reference-named functions over torch CUDA tensors
    layers        Fp8Linear, SmoothQuantLinear, W4A4Gemm (the reference's quantized-Linear layers)
    flux_blocks   FluxSingleTransformerBlockOp, FluxTransformerBlockOp, LyraDiffCommonContext (Python mirrors)
    flux_model    FluxTransformer2DModelOp (Python mirror of the whole-model class)
    torch_classes load(): the same classes registered in C++ as torch.classes.lyradiff.*
    replicas      one copy of the workload per GPU under torch.distributed (no collective on the data path)
    build         python -m lyradiff_b200.build

Submodules are imported on use; importing the package itself loads nothing.
"""
