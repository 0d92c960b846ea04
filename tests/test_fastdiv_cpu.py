"""The reciprocal division the pooling and patch-matrix kernels use (FastDiv in metalhlo_b200/csrc/common.cuh):
mul = ceil(2^(31+s) / d) with s = ceil(log2 d), quotient = (n * mul) >> (32 + s - 1). The formula is restated here and
checked against integer division for every n < 2^31 class that matters (multiples, neighbours of multiples, extremes)."""
import random


def constants(d):
    if d == 1:
        return 0, 0
    s = (d - 1).bit_length()
    mul = -(-(1 << (31 + s)) // d)
    assert mul < (1 << 32), (d, mul)  # fits the 32-bit field
    return mul, s - 1


def fast_div(n, d, mul, shift):
    return n if d == 1 else ((n * mul) >> 32) >> shift


def test_fast_division_matches_integer_division():
    rnd = random.Random(20240607)
    divisors = list(range(1, 3000)) + [rnd.randrange(1, 1 << 31) for _ in range(5000)]
    divisors += [(1 << k) + j for k in range(1, 31) for j in (-1, 0, 1)]
    top = (1 << 31) - 1
    for d in divisors:
        mul, shift = constants(d)
        probes = [0, 1, d - 1, d, d + 1, 2 * d - 1, 2 * d, top, top - 1, top // d * d, top // d * d - 1]
        probes += [rnd.randrange(0, 1 << 31) for _ in range(8)]
        for n in probes:
            if 0 <= n <= top:
                assert fast_div(n, d, mul, shift) == n // d, (n, d)
