"""CPU checks of the oracle's restatement of the operand emitters (llm-1b/emit.cu): internal
consistency only -- the reference holds no CPU implementation or fixture for these kernels."""
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
