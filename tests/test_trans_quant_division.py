"""Host-side proof obligation of the transposing quantiser's division.

The reference divides every element by the block scale in fp32
(quant/trans_per_block_quant_expand_128x.py:216-273, `x / scale`).  The CUDA kernel computes one
correctly rounded reciprocal per block and then, per element,

    q0 = RN(x * r);  e = RN(x - scale * q0);  q1 = RN(q0 + e * r)

with fused multiply-adds.  That sequence is not a correctly rounded division for arbitrary fp32
operands, but here x carries an 8-bit (bf16) or 11-bit (fp16) significand and scale = RN(amax / 448)
with amax of the same format, and fp32 rounding depends on significands only (no underflow is
involved for quotients that matter, which the kernel guarantees by a range check).  So the claim
"q1 == RN(x / scale)" is finite and is checked here for every pair of significands with exact
rational arithmetic.
"""
from fractions import Fraction as F

import pytest


def rn(fr, p=24):
    """Round a rational to the nearest p-bit binary float, ties to even, unbounded exponent."""
    if fr == 0:
        return fr
    sign = 1 if fr > 0 else -1
    n, d = abs(fr).numerator, abs(fr).denominator
    k = n.bit_length() - d.bit_length() - p

    def scaled(k):
        return (n << -k, d) if k < 0 else (n, d << k)

    nn, dd = scaled(k)
    if nn // dd >= (1 << p):
        k += 1
    elif nn // dd < (1 << (p - 1)):
        k -= 1
    nn, dd = scaled(k)
    m, rem = divmod(nn, dd)
    assert (1 << (p - 1)) <= m < (1 << p)
    if 2 * rem > dd or (2 * rem == dd and (m & 1)):
        m += 1
    return sign * F(m) * F(2) ** k


def test_rn_helper():
    assert rn(F(1, 3)) == F(11184811, 2 ** 25)          # 0x3eaaaaab
    assert rn(F(2 ** 24 + 1)) == F(2 ** 24)             # tie -> even
    assert rn(F(2 ** 24 + 3)) == F(2 ** 24 + 4)         # tie -> even (upwards)
    assert rn(F(-5, 2)) == F(-5, 2)


@pytest.mark.parametrize("bits", [8, 11], ids=["bf16", "fp16"])
def test_reciprocal_residual_division_is_correctly_rounded(bits):
    lo, hi = 1 << (bits - 1), 1 << bits
    for amax_sig in range(lo, hi):
        scale = rn(F(amax_sig, 448))
        r = rn(1 / scale)
        for x_sig in range(lo, hi):
            x = F(x_sig)
            q0 = rn(x * r)
            e = rn(x - scale * q0)  # one rounding, as the fused multiply-add does (not always exact)
            q1 = rn(q0 + e * r)
            assert q1 == rn(x / scale), (amax_sig, x_sig)
