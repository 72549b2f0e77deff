"""FP8 e4m3 (the "fn" flavour: no infinities, 0x7F/0xFF = NaN, max finite 448) codec in numpy.

Test infrastructure.  The reference quantizes with ``__nv_fp8_e4m3(float)``
(src/lyradiff/utils/cuda_type_utils.cuh:610-613), i.e. round-to-nearest-even
with saturation to the largest finite value (+-448) instead of overflow to NaN.
The encoder below restates that conversion with integer/power-of-two
arithmetic only, so that it does not depend on any library's float8 cast.
"""

import numpy as np

E4M3_MAX = 448.0


def decode(bits):
    """uint8 e4m3 codes -> float32 values (exact)."""
    b = np.asarray(bits, dtype=np.uint8).astype(np.int32)
    sign = np.where(b & 0x80, -1.0, 1.0).astype(np.float32)
    exp = (b >> 3) & 0xF
    man = b & 0x7
    normal = np.ldexp((8 + man).astype(np.float32), exp - 7 - 3)
    subnormal = np.ldexp(man.astype(np.float32), -9)
    val = np.where(exp == 0, subnormal, normal).astype(np.float32)
    val = np.where((exp == 15) & (man == 7), np.float32(np.nan), val)
    return (sign * val).astype(np.float32)


def encode(x):
    """float32 -> uint8 e4m3 codes: round-half-to-even, saturate to +-448, NaN -> 0x7F."""
    x = np.asarray(x, dtype=np.float32)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    a = np.abs(x).astype(np.float64)
    nan = np.isnan(a)
    a = np.where(nan, 0.0, a)
    a = np.minimum(a, E4M3_MAX)
    # exponent of the binade; frexp gives a = m * 2**e with m in [0.5, 1)
    _, e = np.frexp(a)
    e = e - 1  # now a in [2**e, 2**(e+1))
    e = np.maximum(e, -6)  # below 2**-6 the spacing is the subnormal one
    quantum = np.ldexp(1.0, e - 3)
    q = np.rint(a / quantum)  # exact power-of-two scaling; rint = half-to-even
    v = q * quantum  # representable value (may have carried into the next binade)
    _, e2 = np.frexp(v)
    e2 = e2 - 1
    is_sub = (v < np.ldexp(1.0, -6))
    man_sub = np.rint(v / np.ldexp(1.0, -9)).astype(np.int64)
    e2c = np.maximum(e2, -6)
    man_norm = np.rint(v / np.ldexp(1.0, e2c - 3)).astype(np.int64) - 8
    bits_norm = ((e2c + 7) << 3) | man_norm
    bits = np.where(is_sub, man_sub, bits_norm).astype(np.uint8)
    bits = np.where(v == 0.0, np.uint8(0), bits)
    bits = bits | sign
    bits = np.where(nan, np.uint8(0x7F), bits)
    return bits.astype(np.uint8)
