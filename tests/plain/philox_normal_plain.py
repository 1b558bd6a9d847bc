"""The random-weights generator in plain Python, one element at a time, as the tests'
copy of its definition (the package's numpy version and its CUDA kernel must give these
bits).

value(seed, tensor, element):
  block, lane = divmod(element, 4)
  w = Philox4x32-10(counter (block lo, block hi, tensor, 0x6e6f726d), key (seed lo, seed hi))
  lanes 0,1 take the word pair (w0, w1), lanes 2,3 take (w2, w3); Box-Muller:
  u1 = ((a >> 8) + 1) / 2^24, angle = 2 pi (b >> 8) / 2^24, z = sqrt(-2 ln u1) * (cos | sin)(angle)
with ln, cos and sin computed by short series in which every step is one float32 operation.
"""
import math

import numpy as np

from .philox_plain import philox4x32_10

F = np.float32
TAG = 0x6E6F726D


def _ln_unit(k1: int) -> np.float32:
    """ln(k1 / 2^24) for 1 <= k1 <= 2^24."""
    e = k1.bit_length() - 1
    m = F(k1) / F(2 ** e)                               # exact: a power of two
    s = (m - F(1)) / (m + F(1))
    s2 = s * s
    p = F(1 / 13)
    for k in (11, 9, 7, 5, 3, 1):
        p = p * s2 + F(1 / k)
    return F(e - 24) * F(math.log(2)) + (F(2) * s) * p


def _cos_sin(k2: int):
    """(cos, sin) of 2 pi k2 / 2^24 for 0 <= k2 < 2^24."""
    q = k2 >> 22
    x = (F(k2 & 0x3FFFFF) * F(2.0 ** -22)) * F(math.pi / 2)
    x2 = x * x
    ps = F(-1 / math.factorial(11))
    for k, sign in ((9, 1), (7, -1), (5, 1), (3, -1), (1, 1)):
        ps = ps * x2 + F(sign / math.factorial(k))
    sn = x * ps
    pc = F(1 / math.factorial(12))
    for k, sign in ((10, -1), (8, 1), (6, -1), (4, 1), (2, -1), (0, 1)):
        pc = pc * x2 + F(sign / math.factorial(k))
    return [(pc, sn), (-sn, pc), (-pc, -sn), (sn, -pc)][q]


def standard_normal(seed: int, tensor: int, element: int) -> np.float32:
    block, lane = divmod(element, 4)
    w = philox4x32_10((block & 0xFFFFFFFF, block >> 32, tensor & 0xFFFFFFFF, TAG),
                      (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
    a, b = (w[0], w[1]) if lane < 2 else (w[2], w[3])
    with np.errstate(all="ignore"):
        r = np.sqrt(F(-2) * _ln_unit((a >> 8) + 1))
        c, s = _cos_sin(b >> 8)
        return r * (c if lane % 2 == 0 else s)


def value(seed: int, tensor: int, element: int, kind: str, std: float) -> np.float32:
    """``kind`` "matrix": std * z; "scale": 1 + std * z."""
    v = F(std) * standard_normal(seed, tensor, element)
    return F(1) + v if kind == "scale" else v


def to_bfloat16_bits(x: np.float32) -> int:
    """Round to nearest even on the upper 16 bits (finite values)."""
    u = int(np.float32(x).view(np.uint32))
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF
