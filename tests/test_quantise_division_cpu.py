"""The e4m3 quantiser divides a row's 16 values by the row's scale with ONE correctly rounded reciprocal and a
remainder step (csrc/kv_row.cuh quantise) instead of 16 IEEE divisions. This checks, in exact rational arithmetic, that
the step returns the correctly rounded fp32 quotient for the kernel's whole input domain: x and amax are bf16-valued
(8-bit significands), scale = RN(amax / 448), and |x| <= amax; exponent differences beyond 25 give quotients that e4m3
rounds to zero either way."""

from fractions import Fraction as F


def rn32(v: F) -> F:
    """v rounded to the nearest fp32 value, ties to even (normal range)."""
    if v == 0:
        return F(0)
    sign, a = (1 if v > 0 else -1), abs(v)
    e = a.numerator.bit_length() - a.denominator.bit_length()
    if F(2) ** e > a:
        e -= 1
    if F(2) ** (e + 1) <= a:
        e += 1
    ulp = F(2) ** (e - 23)
    q = a / ulp
    n = q.numerator // q.denominator
    rem = q - n
    if rem > F(1, 2) or (rem == F(1, 2) and n % 2 == 1):
        n += 1
    return sign * n * ulp


def test_shared_reciprocal_quotients_are_correctly_rounded():
    cases = 0
    for am in range(128, 256, 1):  # amax = 1.m, every 8-bit significand
        scale = rn32(F(am, 128) / 448)
        r = rn32(1 / scale)
        for xm in range(128, 256, 3 if am % 4 else 1):  # every x significand for a quarter of the amax values
            for de in range(0, 26):
                if de == 0 and xm > am:
                    continue
                x = F(xm, 128) / (2 ** de)
                q0 = rn32(x * r)
                e = rn32(-scale * q0 + x)  # one fma: a single rounding of the remainder
                assert rn32(e * r + q0) == rn32(x / scale), (am, xm, de)
                cases += 1
    assert cases > 150_000
