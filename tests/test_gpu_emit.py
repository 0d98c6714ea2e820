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
