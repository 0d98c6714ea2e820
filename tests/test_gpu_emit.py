"""GPU parity of the row-operand emitter (per-row FP32 scales) against the oracle's restatement of
llm-1b/emit.cu `row_emit`, and its use through the raw GEMM."""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from tests.gpu_util import make_dy, make_w, make_x, rel_fro, to_dev, u8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def emit():
    from nvfp4_training_b200 import _lib, emit
    _lib.load()
    return emit


def _check(q, ref, T, C):
    codes, sbyte, rs = ref
    assert np.array_equal(u8(q.d), codes)
    assert np.array_equal(O.unswizzle_scales(u8(q.s), T, C // 16), sbyte)
    assert np.array_equal(q.rs.cpu().numpy().view(np.uint32), rs.view(np.uint32))


@pytest.mark.parametrize("T,C,seed", [(128, 256, 0), (256, 2048, 1), (128, 3072, 2), (128, 5632, 3), (128, 11264, 4), (384, 1024, 5)])
def test_row_emit_rn_bit_exact(emit, T, C, seed):
    x = make_x(seed, T, C)
    x[3] = 0.0                                   # an all-zero row: inv = 0, every code 0
    x[5, :16] = 0.0
    q = emit.row_emit(to_dev(x), emit.RowQ(T, C), None)
    _check(q, O.emit_rows(x), T, C)


@pytest.mark.parametrize("T,C", [(128, 2048), (128, 768), (256, 11264)])
@pytest.mark.parametrize("seed,salt", [(1, 0), (0xDEADBEEF, 0x51)])
def test_row_emit_sr_bit_exact_with_the_reference_stream(emit, T, C, seed, salt):
    g = make_dy(T + C, T, C)
    rng = torch.tensor([seed, 0xA6B1], dtype=torch.int64, device="cuda").to(torch.int32)
    q = emit.row_emit(to_dev(g), emit.RowQ(T, C), rng, sr=True, salt=salt)
    _check(q, O.emit_rows(g, seed=seed, sr=True, salt=salt), T, C)


def test_row_emit_strided_rows(emit):
    x = make_x(7, 128, 512)
    big = to_dev(np.concatenate([x, x], axis=1))
    q = emit.row_emit(big[:, 512:], emit.RowQ(128, 512), None)
    _check(q, O.emit_rows(x), 128, 512)


def test_row_emit_sr_mean_of_64_beats_rn(emit):
    """The reference's tensor-level unbiasedness check (llm-1b/test_nvq.py:19-22) on the emitter:
    rel-err of the mean of 64 SR dequantizations <= 1/4 of the RN rel-err."""
    g = make_dy(11, 128, 1024)
    gd = to_dev(g)
    acc = np.zeros_like(g, dtype=np.float64)
    for s in range(64):
        rng = torch.tensor([s + 1, 0], dtype=torch.int32, device="cuda")
        q = emit.row_emit(gd, emit.RowQ(128, 1024), rng, sr=True, salt=3)
        acc += O.emit_rows_dequant(u8(q.d), O.unswizzle_scales(u8(q.s), 128, 64), q.rs.cpu().numpy())
    q = emit.row_emit(gd, emit.RowQ(128, 1024), None)
    rn = rel_fro(O.emit_rows_dequant(u8(q.d), O.unswizzle_scales(u8(q.s), 128, 64), q.rs.cpu().numpy()), g)
    assert rel_fro(acc / 64, g) <= 0.25 * rn


def test_forward_through_raw_gemm_and_row_scales(emit):
    """y = (Q(x) @ Q(W)^T) * rs[:, None] * gs  (llm-1b/emit.py:136-140) against the FP64 product of
    the dequantized operands."""
    T, K, N = 256, 1024, 384
    x, w = make_x(1, T, K), make_w(2, N, K)
    q = emit.row_emit(to_dev(x), emit.RowQ(T, K), None)
    wq = emit.WQ(N, K).refresh(to_dev(w))
    raw = emit.mm_row_w(q, wq).float()
    y = (raw * q.rs[:, None] * wq.gs).cpu().numpy()
    xd = O.emit_rows_dequant(*O.emit_rows(x)).astype(np.float64)
    wc, ws, _, _, wgs = O.quant_w2d(w)
    wd = O.dequant(wc, ws, wgs).astype(np.float64)
    assert rel_fro(y, xd @ wd.T) <= 4e-3


def _rng(seed, signs):
    return torch.tensor([seed, signs], dtype=torch.int64, device="cuda").to(torch.int32)


def _check_cols(q, ref, amax_cur, M, C):
    codes, sbyte, cur = ref
    assert np.array_equal(u8(q.d), codes)
    assert np.array_equal(O.unswizzle_scales(u8(q.s), C, M // 16), sbyte)
    assert amax_cur.view(torch.float32).item() == float(cur)


@pytest.mark.parametrize("M,C,seed", [(256, 128, 0), (512, 384, 1), (2048, 256, 2)])
@pytest.mark.parametrize("margin", [1.0, 1.25, 0.5])
def test_col_emit_rn_bit_exact(emit, M, C, seed, margin):
    """`margin` scales the delayed amax: 1.25 = the usual head-room, 0.5 = a stale amax that is too
    small, so blocks saturate (both sides clamp)."""
    signs = 0x3C5A
    g = make_dy(seed + 40, M, C)
    g[:16, 7] = 0.0                                          # a zero block in one column
    au = np.float32(np.abs(O.rht16_cols(g, signs)).max() * np.float32(margin))
    use = torch.tensor([float(au)], dtype=torch.float32, device="cuda")
    cur = torch.zeros(1, dtype=torch.int32, device="cuda")
    q = emit.col_emit(to_dev(g), emit.ColQ(M, C), use, cur, _rng(0, signs))
    _check_cols(q, O.emit_cols(g, signs, au), cur, M, C)


@pytest.mark.parametrize("seed,salt", [(1, 0), (0x12345678, 0xABC)])
def test_col_emit_sr_bit_exact_with_the_reference_stream(emit, seed, salt):
    M, C, signs = 1024, 256, 0xA6B1
    g = make_dy(77, M, C)
    au = np.float32(np.abs(O.rht16_cols(g, signs)).max() * np.float32(1.1))
    use = torch.tensor([float(au)], dtype=torch.float32, device="cuda")
    cur = torch.zeros(1, dtype=torch.int32, device="cuda")
    q = emit.col_emit(to_dev(g), emit.ColQ(M, C), use, cur, _rng(seed, signs), sr=True, salt=salt)
    _check_cols(q, O.emit_cols(g, signs, au, seed=seed, sr=True, salt=salt), cur, M, C)


def test_wgrad_from_two_column_operands(emit):
    """dW = (Q(H dy)^T Q(H x)) * gsA * gsB (llm-1b/emit.py:148-150): equal to the FP64 product of the
    oracle's dequantized operands (FP32 accumulation tolerance), and close to dy^T x (the RHT cancels
    in the product, so only quantization error remains)."""
    M, N, K, signs = 1024, 256, 384, 0x9D2B
    x, g = make_x(3, M, K, outliers=0), make_dy(4, M, N)
    rng = _rng(5, signs)
    ops = []
    for t in (g, x):
        au = np.float32(np.abs(O.rht16_cols(t, signs)).max())
        use = torch.tensor([float(au)], dtype=torch.float32, device="cuda")
        cur = torch.zeros(1, dtype=torch.int32, device="cuda")
        q = emit.col_emit(to_dev(t), emit.ColQ(M, t.shape[1]), use, cur, rng)
        codes, sbyte, _ = O.emit_cols(t, signs, au)
        ops.append((q, au, O.dequant(codes, sbyte, au / np.float32(2688)).astype(np.float64)))
    (qa, aa, da), (qb, ab, db) = ops
    dw = emit.mm_col(qa, qb).cpu().numpy().astype(np.float64) * float(aa / np.float32(2688)) * float(ab / np.float32(2688))
    assert rel_fro(dw, da @ db.T) <= 1e-5
    assert rel_fro(dw, g.astype(np.float64).T @ x.astype(np.float64)) <= 0.25


def test_row_emit_rejects_bad_arguments(emit):
    from nvfp4_training_b200 import _lib as L
    lib = L.load()
    x = torch.zeros(128, 384, dtype=torch.bfloat16, device="cuda")
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    rs = torch.zeros(128, device="cuda")
    a = lambda T, C, sr, rng: (x.data_ptr(), C, T, C, buf.data_ptr(), buf.data_ptr(), rs.data_ptr(), sr, rng, 0, None)
    assert lib.nvfp4_emit_rows(*a(128, 384, 0, None)) == -2        # C % 256
    assert lib.nvfp4_emit_rows(*a(64, 256, 0, None)) == -2         # T % 128
    assert lib.nvfp4_emit_rows(*a(128, 256, 1, None)) == -1        # SR needs the device seed
    assert lib.nvfp4_emit_rows(*a(0, 256, 0, None)) == 0
