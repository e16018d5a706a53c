"""The quantization kernels compute x / scale as rn(1/scale) followed by two FMA correction steps
(div_by_recip in amct_b200/csrc/common.cuh) and rely on that being the correctly rounded quotient,
i.e. what the reference's torch division produces.  This test replays the sequence in exact
rational arithmetic with a hand-written round-to-nearest-even to binary32, on random operands,
on 8-bit-significand numerators (bf16 data), on scales of the form amax / 127 (where exact ties
are frequent) and on divisors with extreme significands."""
import random
from fractions import Fraction


def rn32(fr):
    """Exact Fraction -> nearest binary32 value (ties to even), normal range."""
    if fr == 0:
        return Fraction(0)
    sign = -1 if fr < 0 else 1
    a = abs(fr)
    e = a.numerator.bit_length() - a.denominator.bit_length()
    if Fraction(2) ** e > a:
        e -= 1
    elif Fraction(2) ** (e + 1) <= a:
        e += 1
    ulp = Fraction(2) ** (e - 23)
    m = a / ulp
    fl = m.numerator // m.denominator
    rem = m - fl
    if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and fl % 2 == 1):
        fl += 1
    return sign * fl * ulp


def fma(a, b, c):
    return rn32(a * b + c)


def div_by_recip(x, s):
    y = rn32(1 / s)
    q0 = rn32(x * y)
    q1 = fma(fma(-s, q0, x), y, q0)
    return q0, fma(fma(-s, q1, x), y, q1)


def rand_f32(rng, bits=24):
    m = (rng.getrandbits(bits - 1) | (1 << (bits - 1))) << (24 - bits)
    return Fraction(m) * Fraction(2) ** (rng.randint(-20, 20) - 23) * rng.choice((1, -1))


def test_fma_sequence_is_the_correctly_rounded_quotient():
    rng = random.Random(1)
    plain_product_wrong = 0
    for i in range(6000):
        kind = i % 4
        if kind == 0:
            x, s = rand_f32(rng), abs(rand_f32(rng))
        elif kind == 1:
            x, s = rand_f32(rng, 8), abs(rand_f32(rng))
        elif kind == 2:
            s = rn32(abs(rand_f32(rng, 8)) / 127)
            x = rand_f32(rng, 8)
        else:
            x = rand_f32(rng)
            m = rng.choice(((1 << 24) - 1, (1 << 24) - 2, (1 << 23) + 1, 1 << 23))
            s = Fraction(m) * Fraction(2) ** (rng.randint(-10, 10) - 23)
        want = rn32(x / s)
        q0, q2 = div_by_recip(x, s)
        assert q2 == want, (x, s)
        plain_product_wrong += q0 != want
    # the uncorrected product x * rn(1/s) is NOT enough (why the correction steps are there)
    assert plain_product_wrong > 100


def test_exact_ties_are_common_for_16bit_data():
    """x / (amax / 127) lands exactly on k + 0.5 for a noticeable share of bf16 inputs, and there the
    sequence returns the tie itself (so that round-half-even then decides as in the reference)."""
    rng = random.Random(2)
    ties = 0
    for _ in range(3000):
        amax = abs(rand_f32(rng, 8))
        s = rn32(amax / 127)
        x = rand_f32(rng, 8)
        _, q = div_by_recip(x, s)
        assert q == rn32(x / s)
        if abs(q) < 128 and (2 * q).denominator == 1 and q.denominator == 2:
            ties += 1
    assert ties > 0
