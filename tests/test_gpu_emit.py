"""GPU parity of the row-operand emitter (per-row FP32 scales) against the oracle's restatement of
llm-1b/emit.cu `row_emit`, and its use through the raw GEMM."""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from tests.gpu_util import make_dy, make_w, make_x, rel_fro, to_dev, u8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=[0, 1], ids=["ring", "warp_per_row"])
def emit(request):
    """Both kernels behind nvfp4_emit_rows: 0 = rows through the TMA-fed shared-memory ring, 1 = warp per row."""
    from nvfp4_training_b200 import _lib, emit
    lib = _lib.load()
    assert lib.nvfp4_emit_rows_set_path(request.param) == 0
    yield emit
    lib.nvfp4_emit_rows_set_path(0)
    _lib.check_status()


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


def test_col_emit_hardware_sr_bit_exact(emit):
    """The hardware stochastic-convert mode of the column emitter against the oracle's model of the convert with this
    library's counter-based words (key from rng[0] ^ salt and the block index)."""
    M, C, signs = 2048, 384, 0xA6B1
    g = make_dy(78, M, C)
    au = np.float32(np.abs(O.rht16_cols(g, signs)).max() * np.float32(1.5))
    use = torch.tensor([float(au)], dtype=torch.float32, device="cuda")
    cur = torch.zeros(1, dtype=torch.int32, device="cuda")
    q = emit.col_emit(to_dev(g), emit.ColQ(M, C), use, cur, _rng(77, signs), sr="hw", salt=5)
    _check_cols(q, O.emit_cols(g, signs, au, seed=77, sr="hw", salt=5), cur, M, C)


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


# ---------------------------------------------------------------------------------------- pins and the fused epilogue
def test_row_emit_against_the_reference_torch_emulation(emit):
    """Cross-check against `q_rows` of small-model/qref.py:15-31 (restated as `O.qref_rows`, itself bit-exact against
    the reference's `model_ref.nvfp4_1d` row by row): the kernel multiplies by reciprocals where the emulation divides,
    so codes / scale bytes may differ where a last-bit difference crosses a rounding boundary.  Stated bound: at most
    2e-3 of the codes and of the scale bytes, never by more than one step; dequantized tensors within 1e-2."""
    for seed, (T, C) in enumerate([(256, 2048), (128, 5632), (128, 11264)]):
        x = make_x(seed, T, C) if seed != 1 else make_dy(seed, T, C)
        q = emit.row_emit(to_dev(x), emit.RowQ(T, C), None)
        qc, qs, gs = O.qref_rows(x)
        cu = O.unpack_codes(u8(q.d))
        sb = O.unswizzle_scales(u8(q.s), T, C // 16)
        diff = cu != qc
        assert diff.mean() <= 2e-3 and (sb != qs).mean() <= 2e-3, (diff.mean(), (sb != qs).mean())
        assert np.abs((cu & 7).astype(int) - (qc & 7).astype(int))[diff].max(initial=0) <= 1
        assert np.abs(sb.astype(int) - qs.astype(int)).max() <= 1
        ref = (O.E2M1_TABLE[qc] * np.repeat(O.e4m3_decode(qs), 16, axis=1)) * gs[:, None]
        assert rel_fro(emit.dequant(q.d, q.s, q.rs).cpu().numpy(), ref) < 1e-2


def test_reference_emit_checks_with_stated_bounds(emit):
    """The quantities llm-1b/test_emit.py:31-46 prints, on its shapes scaled down 8x in tokens, each with a bound:
    row_emit RN error < 0.12 and SR mean(32) error < 0.4 x RN; wgrad from two column operands with a calibrated
    delayed amax (x2 margin) < 0.2 of exact; forward GEMM with per-row scales < 0.15 of exact, dgrad (stochastically
    rounded gradient operand) < 0.2."""
    T, D, F = 1024, 2048, 5632
    g0 = torch.Generator(device="cuda").manual_seed(0)
    rng = torch.tensor([12345, 0b1011001110001101], dtype=torch.int32, device="cuda")
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
    g = torch.randn(T, D, generator=g0, device="cuda").bfloat16()
    qg = emit.RowQ(T, D)
    acc = torch.zeros(T, D, device="cuda")
    for i in range(32):
        rng[0] = i * 7919 + 1
        emit.row_emit(g, qg, rng, sr=True)
        acc += emit.dequant(qg.d, qg.s, qg.rs)
    emit.row_emit(g, qg, rng, sr=False)
    e_rn, e_sr = rel(emit.dequant(qg.d, qg.s, qg.rs), g), rel(acc / 32, g)
    assert e_rn < 0.12 and e_sr < 0.4 * e_rn, (e_rn, e_sr)
    # col_emit + wgrad GEMM, delayed amax calibrated by a first pass
    gg = (torch.randn(T, F, generator=g0, device="cuda") * 1e-3).bfloat16()
    aa = torch.randn(T, D, generator=g0, device="cuda").bfloat16()
    cu = torch.ones(2, device="cuda") * 1e9
    cc = torch.zeros(2, dtype=torch.int32, device="cuda")
    qc1, qc2 = emit.ColQ(T, F), emit.ColQ(T, D)
    emit.col_emit(gg, qc1, cu[0:1], cc[0:1], rng, sr=True)
    emit.col_emit(aa, qc2, cu[1:2], cc[1:2], rng)
    cu.copy_(cc.view(torch.float32) * 2.0)
    cc.zero_()
    emit.col_emit(gg, qc1, cu[0:1], cc[0:1], rng, sr=True, salt=3)
    emit.col_emit(aa, qc2, cu[1:2], cc[1:2], rng)
    dW = emit.mm_col(qc1, qc2).float() * (cu[0] / 2688) * (cu[1] / 2688)
    ref = gg.float().t() @ aa.float()
    assert rel(dW, ref) < 0.2, rel(dW, ref)
    # the same product with the two scales applied in the epilogue, accumulated in place
    dW2 = torch.zeros(F, D, device="cuda")
    emit.mm_col(qc1, qc2, scale=True, amax_a=cu[0:1], amax_b=cu[1:2], out=dW2, accumulate=True)
    assert rel(dW2, dW) < 1e-6
    # weights: forward and dgrad with per-row scales
    W = (torch.randn(F, D, generator=g0, device="cuda") * 0.02).bfloat16()
    wq = emit.WQ(F, D).refresh(W)
    x = torch.randn(T, D, generator=g0, device="cuda").bfloat16()
    hq = emit.row_emit(x, emit.RowQ(T, D), None)
    yraw = emit.mm_row_w(hq, wq)
    yv = yraw.float() * hq.rs[:, None] * wq.gs
    assert rel(yv, x.float() @ W.float().t()) < 0.15
    dq = emit.row_emit(gg, emit.RowQ(T, F), rng, sr=True)
    dx = emit.mm_row_wt(dq, wq).float() * dq.rs[:, None] * wq.gs
    assert rel(dx, gg.float() @ W.float()) < 0.2
    # fused row-scale epilogue == the reference's separate scale_rows pass up to one bf16 rounding of the raw product
    y_fused = emit.mm_row_w(hq, wq, scale=True)
    assert y_fused.dtype == torch.bfloat16 and rel(y_fused, yv) < 3e-3
    assert rel(y_fused, emit.scale_rows(yraw, hq.rs, wq.gs)) < 5e-3
    dx_fused = emit.mm_row_wt(dq, wq, scale=True)
    assert rel(dx_fused, dx) < 3e-3


@pytest.mark.parametrize("tile", [0, 128, 256, 512, 448, 384])
def test_gemm_row_scale_epilogue(emit, tile):
    """alpha[row] = rs[row] * gs in the epilogue of every GEMM variant (one-CTA and CTA-pair kernels, bf16 and FP32,
    accumulate): against the FP64 product of the dequantized operands with the scales applied per row."""
    from nvfp4_training_b200 import _lib as L
    M, N, K = 512, 768, 1024
    x, w = make_x(5, M, K), make_w(6, N, K)
    q = emit.row_emit(to_dev(x), emit.RowQ(M, K), None)
    wq = emit.WQ(N, K).refresh(to_dev(w))
    codes, sbyte, rs = O.emit_rows(x)
    wc, ws, _, _, wgs = O.quant_w2d(w)
    want = O.gemm_unit(codes, sbyte, wc, ws) * rs.astype(np.float64)[:, None] * float(wgs)
    L.load().nvfp4_gemm_force_tile_n(tile)
    try:
        y = emit.mm_row_w(q, wq, scale=True).float().cpu().numpy()
        assert rel_fro(y, want) <= 4e-3
        out = torch.full((M, N), 1.0, device="cuda")
        emit._gemm(q.d, q.s, wq.d, wq.s, out, L.ALPHA_ROW, q.rs, wq.gs, accumulate=True)
        got = out.cpu().numpy().astype(np.float64)
        assert rel_fro(got, want + 1.0) <= 1e-5
        assert (np.abs(got - want - 1.0) <= 1e-4 * np.abs(want) + 1e-5).all()
    finally:
        L.load().nvfp4_gemm_force_tile_n(0)
    L.check_status()


def test_row_emit_ring_many_rows_per_cta_and_hardware_sr():
    """The ring kernel with many rows per CTA (every slot of the ring is reused several times, every consumer warp
    takes several rows): [4096, 2048] round to nearest (whole tensor) and [2048, 11264] with the reference's
    four-sequence dither stream; and the hardware stochastic-rounding mode against the oracle's model of the convert
    with this library's counter-based words."""
    from nvfp4_training_b200 import _lib, emit
    lib = _lib.load()
    assert lib.nvfp4_emit_rows_set_path(0) == 0
    x = make_x(3, 4096, 2048)
    q = emit.row_emit(to_dev(x), emit.RowQ(4096, 2048), None)
    _check(q, O.emit_rows(x), 4096, 2048)
    g = make_dy(4, 2048, 11264)
    rng = torch.tensor([99, 0], dtype=torch.int32, device="cuda")
    q = emit.row_emit(to_dev(g), emit.RowQ(2048, 11264), rng, sr=True, salt=7)
    _check(q, O.emit_rows(g, seed=99, sr=True, salt=7), 2048, 11264)
    g = make_dy(5, 1024, 5632)
    q = emit.row_emit(to_dev(g), emit.RowQ(1024, 5632), rng, sr="hw", salt=11)
    _check(q, O.emit_rows(g, seed=99, sr="hw", salt=11), 1024, 5632)
    # unbiasedness of the hardware mode at tensor level: mean of 64 draws beats round-to-nearest by 4x
    gd = to_dev(g)
    acc = torch.zeros(1024, 5632, device="cuda")
    for s_ in range(64):
        rng[0] = s_ + 1
        qq = emit.row_emit(gd, emit.RowQ(1024, 5632), rng, sr="hw")
        acc += emit.dequant(qq.d, qq.s, qq.rs)
    qq = emit.row_emit(gd, emit.RowQ(1024, 5632), None)
    gf = gd.float()
    e_rn = ((emit.dequant(qq.d, qq.s, qq.rs) - gf).norm() / gf.norm()).item()
    e_sr = ((acc / 64 - gf).norm() / gf.norm()).item()
    assert e_sr <= 0.25 * e_rn, (e_sr, e_rn)
    _lib.check_status()


def test_row_emit_hardware_sr_warp_per_row_and_long_rows():
    """The hardware stochastic-rounding mode through the warp-per-row kernel: forced on a shape the ring kernel also
    takes (same bytes from both), and on rows longer than the ring holds (the LM head's output gradient has 49152
    columns)."""
    from nvfp4_training_b200 import _lib, emit
    lib = _lib.load()
    rng = torch.tensor([41, 0], dtype=torch.int32, device="cuda")
    g = make_dy(6, 256, 5632)
    want = O.emit_rows(g, seed=41, sr="hw", salt=3)
    try:
        for path in (1, 0):
            assert lib.nvfp4_emit_rows_set_path(path) == 0
            q = emit.row_emit(to_dev(g), emit.RowQ(256, 5632), rng, sr="hw", salt=3)
            _check(q, want, 256, 5632)
    finally:
        lib.nvfp4_emit_rows_set_path(0)
    g = make_dy(7, 128, 49152)
    q = emit.row_emit(to_dev(g), emit.RowQ(128, 49152), rng, sr="hw", salt=9)
    _check(q, O.emit_rows(g, seed=41, sr="hw", salt=9), 128, 49152)
    _lib.check_status()
