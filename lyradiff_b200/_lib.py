"""ctypes loader for liblyraq.so, the C-ABI CUDA library.  There is no fallback: if the library is
missing or lacks a symbol the import of the ops fails with a clear error."""

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("LYRAQ_LIB_PATH", os.path.join(_HERE, "liblyraq.so"))

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_size_t = ctypes.c_size_t
c_float = ctypes.c_float
c_double = ctypes.c_double

# name -> (restype, argtypes); mirrors include/lyraq.h declaration by declaration
SIGNATURES = {
    "lyraq_version": (ctypes.c_char_p, []),
    "lyraq_status_string": (ctypes.c_char_p, [c_int]),
    "lyraq_last_status": (c_int, [c_void_p, ctypes.POINTER(ctypes.c_uint32)]),
    "lyraq_debug_force_gemm_tile": (c_int, [c_int]),
    "lyraq_debug_set_dependent_launch": (c_int, [c_int]),
    "lyraq_debug_attention_wait_test": (c_int, [c_int, ctypes.c_uint]),
    "lyraq_last_cuda_error": (ctypes.c_char_p, []),
    "lyraq_debug_set_row_vectors_per_thread": (c_int, [c_int]),
    "lyraq_debug_set_special_row_kernels": (c_int, [c_int]),
    "lyraq_quant_int8": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_size_t, c_size_t, c_void_p]),
    "lyraq_quant_fp8": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_size_t, c_void_p]),
    "lyraq_fp8_amax_scale": (c_int, [c_void_p, c_void_p, c_int, c_size_t, c_void_p]),
    "lyraq_weight_quant_fp8": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_void_p]),
    "lyraq_quant_int4_g64": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_size_t,
                                     c_size_t, c_void_p]),
    "lyraq_weight_quant_int8": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_size_t, c_size_t, c_void_p]),
    "lyraq_weight_quant_int4_g64": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_size_t, c_size_t, c_void_p]),
    "lyraq_adaln_quant": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                  c_void_p, c_size_t, c_size_t, c_size_t, c_double, c_void_p]),
    "lyraq_adaln_quant_fp8x2": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                        c_size_t, c_size_t, c_size_t, c_double, c_void_p]),
    "lyraq_ln_quant_int8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                    c_void_p, c_size_t, c_size_t, c_double, c_void_p]),
    "lyraq_geglu_quant_int8": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_size_t, c_size_t,
                                       c_void_p]),
    "lyraq_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "lyraq_gemm_int8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                                c_int, c_void_p, c_size_t, c_void_p]),
    "lyraq_gemm_int8_residual": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                         c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "lyraq_gemm_fp8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float,
                               c_float, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "lyraq_gemm_fp8_gate": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                    c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "lyraq_gemm_fp8_quant": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                     c_float, c_float, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "lyraq_gemm_fp8_quant_ld": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_int, c_void_p,
                                        c_void_p, c_float, c_float, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "lyraq_gemm_fp8_qk_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_void_p, c_void_p, c_void_p,
                                       c_int, c_int, c_double, c_int, c_int, c_int, c_void_p]),
    "lyraq_rmsnorm_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_double, c_size_t, c_size_t, c_int, c_int,
                                   c_void_p]),
    "lyraq_attention": (c_int, [c_void_p, c_int, c_size_t, c_void_p, c_void_p, c_size_t, c_void_p, c_size_t, c_void_p, c_int,
                                c_size_t, c_size_t, c_int, c_int, c_float, c_void_p]),
    "lyraq_quant_fp8_2d": (c_int, [c_void_p, c_size_t, c_void_p, c_int, c_void_p, c_size_t, c_size_t, c_void_p]),
    "lyraq_load_lora": (c_int, [c_void_p, c_void_p, c_int, c_float, c_size_t, c_void_p]),
    "lyraq_gate_residual": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_size_t, c_size_t, c_void_p]),
    "lyraq_gemm_w4a4": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "lyraq_linear_fp8_forward": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                                         c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "lyraq_linear_int8_forward": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                          c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "lyraq_w4a4_forward": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                   c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "lyraq_w4a4_lora_forward": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "lyraq_w4a4_forward_static": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                          c_int, c_int, c_int, c_int, c_void_p]),
    "lyraq_static_scratch_bytes": (c_size_t, []),
}

_lib = None


class LyraqError(RuntimeError):
    def __init__(self, status, where):
        self.status = status
        msg = lib().lyraq_status_string(status).decode() if _lib is not None else str(status)
        if status == 3 and _lib is not None:
            msg += " [" + lib().lyraq_last_cuda_error().decode() + "]"
        super().__init__("%s failed: %s (status %d)" % (where, msg, status))


def lib():
    """The loaded library with every declared symbol bound and typed."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "liblyraq.so not found at %s; build it with `python -m lyradiff_b200.build` "
                "(there is no CPU or PyTorch fallback)" % LIB_PATH)
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status, where):
    if status != 0:
        raise LyraqError(status, where)
