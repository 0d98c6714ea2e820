"""CPU checks of the oracle's restatement of the operand emitters (llm-1b/emit.cu).  The reference holds no CPU
implementation of these kernels; what pins them here is (a) the reference's torch emulation of per-row-scale
quantization, `q_rows` of small-model/qref.py:15-31, restated as `qref_rows` and itself checked bit for bit against a
fixture made with the reference's `model_ref.nvfp4_1d` row by row, and (b) a stated cross-check between the two forms:
the kernels multiply by reciprocals where the emulation divides, so codes and scale bytes may differ where a last-bit
difference crosses a rounding boundary -- at most 2e-3 of them, never by more than one code step / one scale step."""
import numpy as np

from oracle import nvfp4_oracle as O
from tests.gpu_util import make_dy, make_x, rel_fro


def test_emit_rows_dequantizes_close_to_the_input_and_scales_are_per_row():
    x = make_x(0, 64, 512)
    x[3] = 0.0
    codes, sbyte, rs = O.emit_rows(x)
    assert rs[3] == 0.0 and not codes[3].any() and not sbyte[3].any()
    assert np.array_equal(rs, (np.abs(x).max(axis=1) * np.float32(np.float32(1) / np.float32(2688))).astype(np.float32))
    # every row uses its full range: the largest scale byte of a non-zero row is 448 (0x7E)
    assert (sbyte.max(axis=1)[np.abs(x).max(axis=1) > 0] == 0x7E).all()
    assert rel_fro(O.emit_rows_dequant(codes, sbyte, rs), x) < 0.12


def test_emit_rows_sr_is_unbiased_and_seeded():
    g = make_dy(1, 32, 256)
    a = O.emit_rows(g, seed=5, sr=True, salt=1)
    b = O.emit_rows(g, seed=5, sr=True, salt=1)
    c = O.emit_rows(g, seed=6, sr=True, salt=1)
    assert np.array_equal(a[0], b[0]) and not np.array_equal(a[0], c[0])
    acc = np.zeros_like(g, dtype=np.float64)
    for s in range(32):
        acc += O.emit_rows_dequant(*O.emit_rows(g, seed=s + 1, sr=True))
    rn = rel_fro(O.emit_rows_dequant(*O.emit_rows(g)), g)
    assert rel_fro(acc / 32, g) < 0.4 * rn


def test_emit_cols_uses_the_delayed_amax_and_reports_the_current_one():
    g = make_dy(2, 128, 64)
    signs = 0x5AA5
    t = O.rht16_cols(g, signs)
    cur_true = np.float32(np.abs(t).max())
    codes, sbyte, cur = O.emit_cols(g, signs, cur_true * np.float32(1.25))
    assert cur == cur_true
    deq = O.dequant(codes, sbyte, cur_true * np.float32(1.25) / np.float32(2688)).reshape(64, 8, 16)
    assert rel_fro(deq, t) < 0.12
    # a stale amax that is too small saturates instead of overflowing
    codes2, sbyte2, _ = O.emit_cols(g, signs, cur_true * np.float32(0.25))
    assert sbyte2.max() == 0x7E and (O.unpack_codes(codes2) & 7).max() == 7


def test_lcg_and_dither_primitives():
    s, r = O.lcg_next(np.uint32(1))
    assert int(s) == (1664525 + 1013904223) & 0xFFFFFFFF and int(r) == int(s) ^ (int(s) >> 16)
    # dither with zero bits truncates toward zero on the E2M1 grid; full bits round up
    v = np.array([0.3, 0.74, 1.4, 2.9, 5.9, -0.3, 7.5], dtype=np.float32)
    assert np.array_equal(O.sr2(v, np.uint32(0)), np.array([0.0, 0.5, 1.0, 2.0, 4.0, -0.0, 6.0], dtype=np.float32))
    assert np.array_equal(O.sr2(v, np.uint32(0x3FF800)), np.array([0.5, 1.0, 1.5, 3.0, 6.0, -0.5, 6.0], dtype=np.float32))


def test_qref_rows_equals_the_reference_fake_quant_row_by_row(golden):
    """`qref_rows` (restatement of small-model/qref.py:15-31) dequantizes to exactly what the reference's own
    `model_ref.nvfp4_1d` gives when each row is quantized as a tensor of its own (fixture `rowscale_*`)."""
    x = O.bf16_bits_to_f32(golden["rowscale_x"])
    codes, sbyte, gs = O.qref_rows(x)
    deq = (O.E2M1_TABLE[codes] * np.repeat(O.e4m3_decode(sbyte), 16, axis=1)).astype(np.float32) * gs[:, None]
    assert np.array_equal(deq.astype(np.float32), golden["rowscale_dq"])


def test_emit_rows_against_the_division_form_within_the_stated_mismatch():
    for seed, (T, C) in enumerate([(256, 2048), (256, 3072), (128, 5632)]):
        x = make_x(seed, T, C) if seed != 1 else make_dy(seed, T, C)
        codes, sbyte, rs = O.emit_rows(x)
        qc, qs, gs = O.qref_rows(x)
        cu = O.unpack_codes(codes)
        diff = cu != qc
        assert diff.mean() <= 2e-3 and (sbyte != qs).mean() <= 2e-3
        assert np.abs((cu & 7).astype(int) - (qc & 7).astype(int))[diff].max(initial=0) <= 1
        assert np.abs(sbyte.astype(int) - qs.astype(int)).max() <= 1
        assert np.max(np.abs(gs - rs) / np.maximum(gs, 1e-30)) <= 2.0 ** -23         # am * (1/2688) vs am / 2688
        assert rel_fro(O.emit_rows_dequant(codes, sbyte, rs), (O.E2M1_TABLE[qc] * np.repeat(O.e4m3_decode(qs), 16, axis=1)) * gs[:, None]) < 1e-2


def test_emit_rows_11264_columns_uses_the_four_sequence_stream():
    """For C == 11264 the reference's launcher runs `row_emit_11264` (row_reg<4, 11>, llm-1b/emit.cu:228-260): checked
    against a scalar walk of that kernel's loop for one row -- sequence s of lane l starts at
    hash32(seed ^ salt ^ hash32(r*128 + s*32 + l)) and handles the chunks 4 j + s."""
    rng = np.random.default_rng(3)
    x = O.bf16_bits_to_f32(O.f32_to_bf16_bits((rng.standard_normal((2, 11264)) * 1e-3).astype(np.float32)))
    seed, salt, r = 77, 5, 1
    codes, sbyte, rs = O.emit_rows(x, seed=seed, sr=True, salt=salt)
    am = np.abs(x[r]).max().astype(np.float32)
    inv = np.float32(np.float32(2688.0) / am)
    got = O.unpack_codes(codes)[r]
    for sub in (0, 3):
        for lane in (0, 17):
            st = O.hash32(np.uint32(seed) ^ np.uint32(salt) ^ O.hash32(np.uint32(r * 128 + sub * 32 + lane)))
            for j in range(11):
                col = (j * 4 + sub) * 256 + lane * 8
                blk = x[r, col & ~15:(col & ~15) + 16]
                m = np.abs(blk).max().astype(np.float32)
                sb = O.e4m3_encode(np.float32(np.float32(m * inv) * np.float32(np.float32(1) / np.float32(6))))
                sd = O.e4m3_decode(sb)
                k = np.float32(inv / sd) if sd > 0 else np.float32(0)
                c8, st = O._emit_pack8(x[r, col:col + 8][None, :], np.array([k], dtype=np.float32), True, st)
                assert np.array_equal(np.asarray(c8).reshape(-1), got[col:col + 8]), (sub, lane, j)


def test_fma_f32_is_correctly_rounded():
    """The oracle's fused multiply-add against exact rational arithmetic, including products that sit exactly half-way
    between two float32 values with an addend far below the last bit (where a float64 sum would round the wrong way)."""
    from fractions import Fraction
    rng = np.random.default_rng(0)
    n = 1500
    a = rng.standard_normal(n).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    c = (rng.standard_normal(n) * 10.0 ** rng.integers(-12, 3, n)).astype(np.float32)
    a[:200] = np.float32(1 + 2.0 ** -12)
    b[:200] = np.float32(1 + 2.0 ** -12)          # product 1 + 2^-11 + 2^-24: a midpoint of the float32 grid
    c[:100] = np.float32(2.0 ** -60)
    c[100:200] = np.float32(-2.0 ** -60)
    r = O.fma_f32(a, b, c)
    for i in range(n):
        v = Fraction(float(a[i])) * Fraction(float(b[i])) + Fraction(float(c[i]))
        f = np.float32(float(v))
        cands = [np.nextafter(f, np.float32(-np.inf)), f, np.nextafter(f, np.float32(np.inf))]
        best = min(cands, key=lambda t: (abs(Fraction(float(t)) - v), int(np.float32(t).view(np.uint32)) & 1))
        assert np.float32(best).view(np.uint32) == r[i].view(np.uint32), i
    assert r[0] > r[150]


def test_fused_producers_self_consistency():
    """rms_emit / swiglu_emit of the oracle: the operand dequantizes back to the FP32 values it was made from within
    one code step of each block, rstd matches the plain formula, the residual is bf16; mom_acc is unbiased."""
    rng = np.random.default_rng(1)
    bf = lambda v: O.bf16_round(np.asarray(v, dtype=np.float32))
    T, D = 16, 2048
    x, y = bf(rng.standard_normal((T, D))), bf(rng.standard_normal((T, D)) * 40)
    ys, ygw, w = (0.01 + 0.02 * rng.random(T)).astype(np.float32), np.float32(0.7), bf(1 + 0.1 * rng.standard_normal(D))
    o = O.rms_emit(x, w, y, ys, ygw)
    xn = x.astype(np.float64) + y.astype(np.float64) * (ys * ygw).astype(np.float64)[:, None]
    assert np.array_equal(o["xout"], bf(o["xout"])) and np.abs(o["xout"] - xn).max() <= np.abs(xn).max() * 2.0 ** -8
    want = 1 / np.sqrt((o["xout"].astype(np.float64) ** 2).mean(axis=1) + 1e-5)
    assert np.abs(o["rstd"] / want - 1).max() < 1e-6
    step = np.repeat(O.e4m3_decode(o["scales"]) * o["rs"][:, None], 16, axis=1)
    assert (np.abs(O.emit_rows_dequant(o["codes"], o["scales"], o["rs"]) - o["h"]) <= step + 1e-12).all()
    gu = bf(rng.standard_normal((T, 1024)) * 3)
    s = O.swiglu_emit(gu, np.full(T, 0.5, np.float32), 1.5)
    step = np.repeat(O.e4m3_decode(s["scales"]) * s["rs"][:, None], 16, axis=1)
    assert (np.abs(O.emit_rows_dequant(s["codes"], s["scales"], s["rs"]) - s["a"]) <= step + 1e-12).all()
    m, g = bf(rng.standard_normal(4096) * 0.1), bf(rng.standard_normal(4096) * 1e-3)
    acc = sum(O.mom_acc(m, g, 0.5, 0.5, seed, 3).astype(np.float64) for seed in range(1, 65)) / 64
    exact = m.astype(np.float64) + 0.25 * g.astype(np.float64)
    assert np.mean(np.abs(acc - exact) / (np.abs(exact) * 2.0 ** -8)) < 0.15


def test_qref_rows_gs_equals_the_reference_formula(golden):
    """`qref_rows_gs` (restatement of `q_rows_gs`, small-model/qref.py:33-42) against the fixture made with the
    reference's own `e4m3` / `fp4_round` and a given per-row scale (twice the row's own; 1.0 for the zero row)."""
    x = O.bf16_bits_to_f32(golden["rowscale_x"])
    gs = golden["rowscale_gs"]
    codes, sbyte = O.qref_rows_gs(x, gs)
    T, C = x.shape
    deq = (O.E2M1_TABLE[codes].reshape(T, C // 16, 16) * O.e4m3_decode(sbyte)[:, :, None]).astype(np.float32).reshape(T, C)
    deq = (deq * gs[:, None]).astype(np.float32)
    assert np.array_equal(deq, golden["rowscale_gs_dq"])
    # with the row's own scale it is `qref_rows`
    c2, s2, g2 = O.qref_rows(x)
    own = np.where(g2 > 0, g2, np.float32(1))
    c3, s3 = O.qref_rows_gs(x, own)
    assert np.array_equal(c2, c3) and np.array_equal(s2, s3)
