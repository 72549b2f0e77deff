"""CPU tests of the drop-in boundary: the C-ABI library loads, exports every symbol the header
declares, and refuses bad arguments before touching a device (no compute call is made here)."""

import ctypes
import os
import re

import pytest

from lyradiff_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "lyraq.h")


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.lib()


def declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"LYRAQ_API[^;(]*?\b(lyraq_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for required in ("lyraq_quant_int8", "lyraq_quant_fp8", "lyraq_quant_int4_g64", "lyraq_adaln_quant",
                     "lyraq_ln_quant_int8", "lyraq_geglu_quant_int8", "lyraq_gemm_int8", "lyraq_gemm_fp8",
                     "lyraq_gemm_w4a4", "lyraq_weight_quant_int8", "lyraq_weight_quant_int4_g64",
                     "lyraq_fp8_amax_scale", "lyraq_workspace_bytes", "lyraq_last_status"):
        assert required in names


def test_library_exports_every_declared_symbol(lib):
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(raw, name), name


def test_python_signatures_cover_the_header(lib):
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_every_declaration_cites_the_reference():
    text = open(HEADER).read()
    # each entry point's comment either names a reference file:line or says there is no counterpart
    blocks = re.findall(r"/\*((?:(?!\*/).)*?)\*/\s*LYRAQ_API[^;]*?\b(lyraq_\w+)\s*\(", text, flags=re.S)
    assert len(blocks) >= 14
    for comment, name in blocks:
        assert ("src/lyradiff" in comment or "lyradiff/" in comment or "no counterpart" in comment
                or "int8_gemm_template.h" in comment), name


def test_status_strings_and_version(lib):
    assert lib.lyraq_version().decode().startswith("lyraq")
    assert lib.lyraq_status_string(0) == b"ok"
    assert b"unknown" in lib.lyraq_status_string(99)
    assert lib.lyraq_workspace_bytes(0, 128, 128, 128) == 0


def test_bad_arguments_are_refused_without_a_device(lib):
    INVALID, UNSUPPORTED = 1, 2
    # null pointers
    assert lib.lyraq_quant_int8(None, None, 0, None, None, 0, 4, 64, None) == INVALID
    assert lib.lyraq_quant_fp8(None, None, 1, None, 1, 64, None) == INVALID
    assert lib.lyraq_gemm_int8(None, None, None, None, 0, None, 0, None, 128, 128, 128, None, 0, None) == INVALID
    assert lib.lyraq_gemm_fp8(None, None, None, None, None, 1, None, None, 1.0, 0.0, 0, 128, 128, 128, None, 0, None) == INVALID
    assert lib.lyraq_gemm_w4a4(None, None, None, None, 2, None, 1, None, 2, None, None, None, 0, 128, 128, 128, None, 0, None) == INVALID
    # fake but well-aligned addresses: shape checks come before any launch
    p = 0x1000
    assert lib.lyraq_quant_int8(p, p, 0, None, p, 0, 4, 60, None) == UNSUPPORTED       # dim % 8
    assert lib.lyraq_quant_int8(p, p, 0, None, p, 0, 4, 32768, None) == UNSUPPORTED    # dim too large
    assert lib.lyraq_quant_int8(p, p, 2, None, p, 0, 4, 64, None) == UNSUPPORTED       # fp32 source
    assert lib.lyraq_quant_int8(p, p + 2, 0, None, p, 0, 4, 64, None) == INVALID       # misaligned source
    assert lib.lyraq_quant_int8(p, p, 0, None, p, 7, 4, 64, None) == INVALID           # bad scale mode
    assert lib.lyraq_quant_int4_g64(p, p, None, p, 1, None, None, 4, 96, None) == UNSUPPORTED  # k % 64
    assert lib.lyraq_gemm_int8(p, p, p, p, 0, p, 0, None, 128, 128, 120, None, 0, None) == UNSUPPORTED  # k % 16
    assert lib.lyraq_gemm_int8(p, p, p, p, 5, p, 0, None, 128, 128, 128, None, 0, None) == INVALID
    assert lib.lyraq_gemm_fp8(p, p, p, p, p, 3, None, None, 1.0, 0.0, 0, 128, 128, 128, None, 0, None) == INVALID
    assert lib.lyraq_gemm_w4a4(p, p, p, p, 2, p, 1, None, 2, None, None, None, 0, 128, 128, 96, None, 0, None) == UNSUPPORTED
    # the kernels between the linears of a block
    assert lib.lyraq_rmsnorm_rope(None, None, None, None, 1, 1e-6, 1, 8, 2, 128, None) == INVALID
    assert lib.lyraq_rmsnorm_rope(p, p, p, p, 1, 1e-6, 1, 8, 2, 96, None) == UNSUPPORTED      # head_dim 64 or 128 only
    assert lib.lyraq_rmsnorm_rope(p, p, p, p, 2, 1e-6, 1, 8, 2, 128, None) == UNSUPPORTED     # fp32
    assert lib.lyraq_rmsnorm_rope(p, p, p, p, 1, 1e-6, 0, 8, 2, 128, None) == 0               # empty
    assert lib.lyraq_quant_fp8_2d(p, 64, p, 1, p, 4, 128, None) == INVALID                    # row pitch below the width
    assert lib.lyraq_quant_fp8_2d(p, 256, p, 1, p, 4, 100, None) == UNSUPPORTED               # cols % 8
    assert lib.lyraq_gate_residual(p, p, None, p, 1, 1, 8, 256, None) == INVALID
    assert lib.lyraq_gate_residual(p, p, p, p, 1, 1, 8, 100, None) == UNSUPPORTED             # dim % 8
    assert lib.lyraq_gemm_fp8_quant_ld(p, p, p, p, p, 64, p, 1, None, None, 1.0, 0.0, 0, 128, 128, 128, None, 0, None) == INVALID
    assert lib.lyraq_gemm_fp8_quant_ld(p, p, p, p, p, 256, p, 1, None, p, 1.0, 1.0, 0, 128, 128, 128, None, 0, None) == UNSUPPORTED
    assert lib.lyraq_weight_quant_fp8(None, p, p, 1, 64, None) == INVALID
    assert lib.lyraq_gemm_int8_residual(p, p, p, p, 0, p, 3, None, p, 128, 128, 128, None, 0, None) == INVALID  # no int32 form
    # empty problems are a no-op
    assert lib.lyraq_gemm_int8(p, p, p, p, 0, p, 0, None, 0, 128, 128, None, 0, None) == 0
    assert lib.lyraq_quant_fp8(p, p, 1, p, 1, 0, None) == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError):
        _lib.lib()


def test_cpp_shim_compiles_against_the_reference_call_forms():
    """include/lyradiff_shim.h keeps the reference's function names and argument lists: a translation unit that calls
    them the way the reference's layers do must compile (syntax check only, nothing is linked or run)."""
    import shutil
    import subprocess
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    if shutil.which("g++") is None or not os.path.exists(os.path.join(cuda_inc, "cuda_runtime.h")):
        pytest.skip("g++ or CUDA headers not present")
    src = os.path.join(ROOT, "tests", "shim_compile_check.cpp")
    r = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), "-I", cuda_inc, src],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
