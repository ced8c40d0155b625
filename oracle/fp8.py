"""E4M3 (float8_e4m3fn) encode/decode in plain numpy.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

The reference casts with Triton's ``.to(float8e4nv)`` (src/open_vc_attn/quantization.py:188,
src/open_vc_attn/preparation.py:46,78), which on the GPU is the hardware
round-to-nearest-even, saturating conversion.  The values reaching the cast are
already clamped to [-448, 448], so saturation never triggers; the function
below still saturates so that it is total.
"""

import numpy as np

_F32 = np.float32


def _decode_table():
    table = np.zeros(256, dtype=np.float64)
    for code in range(256):
        sign = -1.0 if code & 0x80 else 1.0
        exp = (code >> 3) & 0xF
        man = code & 0x7
        if exp == 0xF and man == 0x7:
            value = np.nan
        elif exp == 0:
            value = man * 2.0**-9
        else:
            value = (1.0 + man / 8.0) * 2.0 ** (exp - 7)
        table[code] = sign * value
    return table


E4M3_DECODE = _decode_table()
E4M3_DECODE_F32 = E4M3_DECODE.astype(np.float32)


def e4m3_decode(codes):
    """uint8 codes -> float32 values (exact)."""
    return E4M3_DECODE_F32[np.asarray(codes, dtype=np.uint8)]


def e4m3_encode(values):
    """float32 -> uint8 E4M3 codes, round-to-nearest-even, saturating at 448."""
    x = np.asarray(values, dtype=np.float32)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    a = np.minimum(np.abs(x).astype(np.float64), 448.0)
    # Quantum of the binade holding a: 2^(e-3) for normals (e >= -6), 2^-9 below.
    _, e = np.frexp(a)  # a = m * 2^e with m in [0.5, 1)  ->  floor(log2 a) = e - 1
    exponent = np.where(a < 2.0**-6, -6, e - 1)
    quantum = np.ldexp(1.0, exponent - 3)
    steps = np.rint(a / quantum)  # RNE; exact because quantum is a power of two
    # steps is in [0, 16]: 16 means a carry into the next binade, which the
    # integer code arithmetic below absorbs (mantissa overflow increments exponent).
    code = np.where(
        exponent == -6,
        steps,  # subnormals and the first normal binade share the 2^-9 quantum
        (exponent + 7) * 8 + (steps - 8),
    )
    code = np.where(np.isnan(x), 0x7F, code).astype(np.uint8)
    return (code | sign).astype(np.uint8)
