"""Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2,
3", 2011) in plain Python, as the tests' copy of the sampler's random stream:
key = (seed_lo, seed_hi), counter = (draws, stream, 0, 0), r = (word0 >> 8) / 2^24."""

M0, M1 = 0xD2511F53, 0xCD9E8D57
W0, W1 = 0x9E3779B9, 0xBB67AE85
MASK = 0xFFFFFFFF


def philox4x32_10(counter, key):
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for _ in range(10):
        p0, p1 = M0 * c0, M1 * c2
        hi0, lo0, hi1, lo1 = p0 >> 32, p0 & MASK, p1 >> 32, p1 & MASK
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & MASK, lo1, (hi0 ^ c3 ^ k1) & MASK, lo0
        k0, k1 = (k0 + W0) & MASK, (k1 + W1) & MASK
    return c0, c1, c2, c3


def uniform(seed: int, stream: int, draw: int) -> float:
    """The draw-th uniform number of a sequence's stream, in [0, 1)."""
    out = philox4x32_10((draw & MASK, stream & MASK, 0, 0), (seed & MASK, (seed >> 32) & MASK))
    return (out[0] >> 8) / 16777216.0
