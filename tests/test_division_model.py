"""CPU check of the arithmetic the quantizer kernels rely on: a/b formed as q0 = RN(a*rb),
rem = a - q0*b (one FMA), q = RN(q0 + rem*rb) with rb = RN(1/b) equals the IEEE quotient for the
divisors the kernels use (tensor scales amax/2688, E4M3 block scales, 6).  The FMA is emulated in
float64 (a product of two float32 values is exact there)."""
import numpy as np

from oracle import nvfp4_oracle as O

f32 = np.float32


def _fma(a, b, c):
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(np.float32)


def _div_by(a, b):
    b = np.broadcast_to(np.asarray(b, dtype=f32), a.shape)
    rb = (f32(1) / b).astype(f32)
    q0 = (a * rb).astype(f32)
    nrem = _fma(q0, b, -a)
    return _fma(-nrem, rb, q0)


def _same_bits(a, b):
    return np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_fma_division_matches_ieee_for_tensor_scales():
    rng = np.random.default_rng(0)
    v = O.bf16_bits_to_f32(rng.integers(0, 1 << 16, 1 << 20).astype(np.uint16))
    v = v[np.isfinite(v) & (np.abs(v) < 1e30) & ((np.abs(v) > 1e-30) | (v == 0))]
    for am in [f32(1.0), f32(4.53125), f32(5.84375), f32(2688.0), f32(0.0123291015625), f32(37.75)]:
        gs = f32(am / f32(2688))
        assert _same_bits(_div_by(v, gs), (v / gs).astype(f32))


def test_fma_division_matches_ieee_for_block_scales_and_six():
    rng = np.random.default_rng(1)
    q = rng.uniform(0, 2688, 1 << 20).astype(f32) * rng.choice([-1, 1], 1 << 20).astype(f32)
    e4 = O.e4m3_decode(np.arange(1, 127, dtype=np.uint8)).astype(f32)
    b = e4[rng.integers(0, e4.size, q.size)]
    assert _same_bits(_div_by(q, b), (q / b).astype(f32))
    assert _same_bits(_div_by(q, f32(6)), (q / f32(6)).astype(f32))


def test_fma_division_keeps_the_sign_of_zero():
    a = np.array([0.0, -0.0], dtype=f32)
    got = _div_by(a, f32(0.0017))
    assert _same_bits(got, a)


def test_tensor_scale_never_has_all_ones_significand():
    """RN(amax/2688) cannot be 2^(e+1) - ulp: the two floats around 2688 * that value map to
    2^(e+1) and 2^(e+1) - 2 ulp."""
    for e in (100, 120, 127, 130, 140):
        top = np.array([((e + 11) << 23) | 0x280000], dtype=np.uint32)   # 1.3125 * 2^(e+11-127)
        ams = (top[0] + np.arange(-4, 5)).astype(np.uint32).view(f32)
        gs = (ams / f32(2688)).astype(f32)
        assert not np.any((gs.view(np.uint32) & 0x7FFFFF) == 0x7FFFFF)


def _rn32(fr):
    """Round a Fraction to the nearest-even float32 (normal range)."""
    from fractions import Fraction as Fr
    import math
    if fr == 0:
        return f32(0)
    s, a = (-1 if fr < 0 else 1), abs(fr)
    e = math.floor(math.log2(a))
    while Fr(2) ** e > a:
        e -= 1
    while Fr(2) ** (e + 1) <= a:
        e += 1
    q = a / Fr(2) ** (e - 23)
    n = q.numerator // q.denominator
    rem = q - n
    if rem > Fr(1, 2) or (rem == Fr(1, 2) and n % 2 == 1):
        n += 1
    return f32(s * float(n) * 2.0 ** (e - 23))


def test_two_word_reciprocal_division_by_block_scale_gives_the_same_codes():
    """The kernels divide by the block scale as RN(t*rh + RN(t*rl)) with rh = RD(1/bs) (rounded down, so that rl >= 0
    and a zero numerator keeps its sign through the sum), rl = RN((1 - rh*bs)*rh).
    A code only depends on how the quotient compares with the seven rounding boundaries b; RN(t/bs) is below,
    on or above b exactly when t is below, on or above c = b*bs.  Exhaustively (exact rational arithmetic): for
    every scale byte and boundary the form maps pred(c), c, succ(c) below, onto and above b -- and so does the
    IEEE division.  Both are monotone in t, hence the same codes for every t."""
    from fractions import Fraction as Fr
    bounds = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
    for sb in range(1, 127):
        bs = O.e4m3_decode(np.array([sb], dtype=np.uint8))[0]
        rh = f32(1.0) / bs
        if Fr(float(rh)) * Fr(float(bs)) > 1:
            rh = np.nextafter(rh, f32(0))                                         # round down
        res = _rn32(Fr(1) - Fr(float(rh)) * Fr(float(bs)))
        assert res >= 0
        assert Fr(float(res)) == Fr(1) - Fr(float(rh)) * Fr(float(bs))            # the residual FMA is exact
        rl = _rn32(Fr(float(res)) * Fr(float(rh)))
        for b in bounds:
            c = f32(b * bs)
            assert Fr(float(c)) == Fr(b) * Fr(float(bs))
            for t, rel in ((np.nextafter(c, f32(0)), -1), (c, 0), (np.nextafter(c, f32(np.inf)), 1)):
                w = _rn32(Fr(float(t)) * Fr(float(rl)))
                y = _rn32(Fr(float(t)) * Fr(float(rh)) + Fr(float(w)))
                assert np.sign(float(y) - b) == rel, (sb, b, rel)
                assert np.sign(float(f32(t / bs)) - b) == rel, (sb, b, rel)
        # signed zeros: the kernel feeds the NEGATED numerator and both words negated; -0 -> +0 and +0 -> -0 in, sign out
        for t in (f32(0.0), f32(-0.0)):
            nt, nrh, nrl = f32(-t), f32(-rh), f32(-rl)
            w = f32(nt * nrl)
            y = f32(np.float64(nt) * np.float64(nrh) + np.float64(w))
            assert np.signbit(y) == np.signbit(t)
