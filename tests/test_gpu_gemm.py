"""GPU parity of the tcgen05 block-scaled FP4 GEMM against an FP32/FP64 matmul of the dequantized
operands (llm-1b/test_nvq.py:12, small-model/test_fp4ops.py:23-27).

Stated tolerances (every product is exact in FP32; only the accumulation order differs):
  FP32 output:  ||C - Y||_F / ||Y||_F <= 1e-5   and   |C - Y| <= 1e-4 |Y| + 1e-6 max|Y|
  bf16 output:  ||C - Y||_F / ||Y||_F <= 4e-3   and   |C - Y| <= 2^-8 |Y| + 1e-6 max|Y|
"""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from tests.gpu_util import make_dy, make_w, make_x, rel_fro, to_dev, u8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mods():
    from nvfp4_training_b200 import _lib, fp4ops, nvq
    _lib.load()
    yield nvq, fp4ops, _lib
    _lib.load().nvfp4_gemm_force_tile_n(0)
    _lib.check_status()


def ref_product(qa, qb, nvq):
    """float64 matmul of the dequantized operands, from the bytes the GPU produced."""
    R, C = qa.d.shape[0], qa.d.shape[1] * 2
    N = qb.d.shape[0]
    sa = O.unswizzle_scales(u8(qa.s), R, C // 16)
    sb = O.unswizzle_scales(u8(qb.s), N, C // 16)
    unit = O.gemm_unit(u8(qa.d), sa, u8(qb.d), sb)
    return unit * (float(qa.gs.item()) * float(qb.gs.item()))


def check_close(c, y, bf16):
    c = c.float().cpu().numpy().astype(np.float64)
    fro, rel = (4e-3, 2.0 ** -8) if bf16 else (1e-5, 1e-4)
    assert rel_fro(c, y) <= fro, rel_fro(c, y)
    bound = rel * np.abs(y) + 1e-6 * np.abs(y).max()
    bad = np.abs(c - y) > bound
    assert not bad.any(), (int(bad.sum()), float(np.abs(c - y).max()))


SHAPES = [(128, 128, 64), (128, 128, 256), (128, 256, 320), (256, 384, 1024), (512, 384, 1024),
          (384, 512, 2048), (128, 768, 4096), (256, 256, 64), (256, 512, 832), (512, 768, 2048), (1024, 256, 4096), (256, 640, 576), (512, 1152, 1024)]


# tiles 512 / 448 / 384 = the CTA-pair kernel with 256- / 192- / 128-wide tiles (needs M a multiple of 256)
@pytest.mark.parametrize("tile", [0, 128, 256, 512, 448, 384])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_mm_vs_dequant_matmul(mods, M, N, K, tile):
    nvq, _, L = mods
    L.load().nvfp4_gemm_force_tile_n(tile)
    qa = nvq.quant_rows(to_dev(make_x(M + K, M, K)))
    qb = nvq.quant_rows(to_dev(make_w(N, N, K)))
    y = ref_product(qa, qb, nvq)
    check_close(nvq.mm(qa, qb, out_dtype=torch.float32), y, bf16=False)
    check_close(nvq.mm(qa, qb), y, bf16=True)
    raw, alpha = nvq.mm(qa, qb, out_dtype=torch.float32, scale=False)
    check_close(raw * alpha, y, bf16=False)
    L.check_status()


def test_mm_identity_scales_exact(mods):
    """Codes in {0, +-0.5, +-1}, all block scales 1, gs 1: every partial sum is a small multiple of
    0.25, so the FP32 result must be exact whatever the accumulation order."""
    nvq, _, L = mods
    rng = np.random.default_rng(0)
    M, N, K = 256, 256, 512
    def mk(R):
        codes = rng.choice(np.array([0, 1, 2, 9, 10], dtype=np.uint8), (R, K))
        d = torch.from_numpy(O.pack_codes(codes)).cuda()
        s = torch.full((R * K // 16,), 0x38, dtype=torch.uint8, device="cuda")     # E4M3 1.0
        return nvq.Q(d.view(torch.float4_e2m1fn_x2), s.view(torch.float8_e4m3fn), torch.ones(1, device="cuda")), codes
    (qa, ca), (qb, cb) = mk(M), mk(N)
    y = O.E2M1_TABLE[ca].astype(np.float64) @ O.E2M1_TABLE[cb].astype(np.float64).T
    for tile in (128, 256, 512, 448, 384):
        L.load().nvfp4_gemm_force_tile_n(tile)
        c = nvq.mm(qa, qb, out_dtype=torch.float32).cpu().numpy()
        assert np.array_equal(c.astype(np.float64), y)
    L.check_status()


def test_mm_scale_layout_per_row_and_kblock(mods):
    """One distinct scale byte per (row, 16-block) on unit codes: pins the swizzled scale layout,
    the shared-memory -> tensor-memory copy and the scale addressing of every K chunk."""
    nvq, _, L = mods
    M, N, K = 256, 256, 512
    rng = np.random.default_rng(1)
    def mk(R):
        codes = np.full((R, K), 2, dtype=np.uint8)                       # +1.0 everywhere
        sc = rng.integers(0x28, 0x48, (R, K // 16), dtype=np.uint8)      # 2^-2 .. 2^2 with mantissas
        d = torch.from_numpy(O.pack_codes(codes)).cuda()
        s = torch.from_numpy(O.swizzle_scales(sc)).cuda()
        return nvq.Q(d.view(torch.float4_e2m1fn_x2), s.view(torch.float8_e4m3fn), torch.ones(1, device="cuda")), sc
    (qa, sa), (qb, sb) = mk(M), mk(N)
    y = 16.0 * (O.e4m3_decode(sa).astype(np.float64) @ O.e4m3_decode(sb).astype(np.float64).T)
    for tile in (128, 256, 512, 448, 384):
        L.load().nvfp4_gemm_force_tile_n(tile)
        check_close(nvq.mm(qa, qb, out_dtype=torch.float32), y, bf16=False)
        check_close(nvq.mm(qa, qb), y, bf16=True)
    L.check_status()


@pytest.mark.parametrize("tile", [0, 512, 448, 384])
def test_mm_accumulate_into_out(mods, tile):
    nvq, _, L = mods
    L.load().nvfp4_gemm_force_tile_n(tile)
    M, N, K = 256, 512, 1024
    qa = nvq.quant_rows(to_dev(make_x(1, M, K)))
    qb = nvq.quant_rows(to_dev(make_w(2, N, K)))
    y = ref_product(qa, qb, nvq)
    out = torch.ones(M, N, device="cuda")
    nvq.mm(qa, qb, out_dtype=torch.float32, out=out, accumulate=True)
    nvq.mm(qa, qb, out_dtype=torch.float32, out=out, accumulate=True)
    check_close(out, 2 * y + 1, bf16=False)
    L.check_status()


@pytest.mark.parametrize("splitk", [2, 5])
def test_pair_kernel_splitk(mods, splitk):
    """Split-K through the CTA-pair kernel: K slices added atomically into a zeroed FP32 output."""
    _, fp4ops, L = mods
    L.load().nvfp4_gemm_force_tile_n(512)
    M, N, K = 256, 512, 2304
    a = fp4ops.quant_rows(to_dev(make_x(5, M, K, outliers=0)))
    b = fp4ops.quant_rows(to_dev(make_x(6, N, K, outliers=0)))
    y = (fp4ops.dequant(a).double() @ fp4ops.dequant(b).double().t()).cpu().numpy()
    check_close(fp4ops.gemm(a, b, splitk=splitk), y, bf16=False)
    L.check_status()


@pytest.mark.parametrize("M,N,K", [(256, 256, 8192), (768, 512, 4096), (512, 384, 16384)])
def test_mm_library_chosen_splitk(mods, M, N, K):
    """splitk = 0: few output tiles and a long contraction, so the library slices K; overwrite (it zero-fills the
    output itself, here pre-filled with garbage) and accumulate (adds to what is there)."""
    nvq, _, L = mods
    qa = nvq.quant_rows(to_dev(make_x(M + K, M, K)))
    qb = nvq.quant_rows(to_dev(make_w(N, N, K)))
    y = ref_product(qa, qb, nvq)
    out = torch.full((M, N), 7.0, device="cuda")
    nvq.mm(qa, qb, out_dtype=torch.float32, out=out, splitk=0)
    check_close(out, y, bf16=False)
    out.fill_(1.0)
    nvq.mm(qa, qb, out_dtype=torch.float32, out=out, accumulate=True, splitk=0)
    nvq.mm(qa, qb, out_dtype=torch.float32, out=out, accumulate=True, splitk=0)
    check_close(out, 2 * y + 1, bf16=False)
    check_close(nvq.mm(qa, qb, splitk=0), y, bf16=True)       # bf16 output: never sliced
    L.check_status()


@pytest.mark.parametrize("splitk", [1, 3, 16])
def test_fp4ops_gemm_splitk_and_strides(mods, splitk):
    """small-model/test_fp4ops.py:23-37 and bench_wgrad.py: linear scales, strided d/s views,
    FP32 split-K accumulation into `out`."""
    _, fp4ops, L = mods
    L.load().nvfp4_gemm_force_tile_n(0)
    M, N, K = 128, 512, 4096
    a = fp4ops.quant_rows(to_dev(make_x(3, M, K, outliers=0)))
    b = fp4ops.quant_rows(to_dev(make_x(4, N, K, outliers=0)))
    y = (fp4ops.dequant(a).double() @ fp4ops.dequant(b).double().t()).cpu().numpy()
    if splitk == 1:
        check_close(fp4ops.gemm(a, b), y, bf16=True)
    else:
        check_close(fp4ops.gemm(a, b, splitk=splitk), y, bf16=False)
    # padded (strided) operand views, accumulate into a pre-filled out
    pad = 144
    def strided(q):
        d = torch.zeros(q.d.shape[0], q.d.shape[1] + pad, dtype=torch.uint8, device="cuda")
        s = torch.zeros(q.s.shape[0], q.s.shape[1] + pad, dtype=torch.uint8, device="cuda")
        d[:, :q.d.shape[1]] = q.d
        s[:, :q.s.shape[1]] = q.s
        return fp4ops.Q(d[:, :q.d.shape[1]], s[:, :q.s.shape[1]], q.amax, q.k)
    out = torch.full((M, N), 2.0, device="cuda")
    fp4ops.gemm(strided(a), strided(b), out=out, splitk=splitk)
    check_close(out, y + 2, bf16=False)
    L.check_status()


def test_wgrad_rht_sr_close_to_exact(mods):
    """llm-1b/test_nvq.py:14-18: dW from RHT + SR operands vs the exact g^T x.  Stated bound: 0.2
    relative Frobenius error (FP4 quantization noise), and equality with the dequant product."""
    nvq, _, L = mods
    M, N, K = 1024, 384, 512
    g = make_dy(7, M, N)
    x = make_x(8, M, K, outliers=0)
    signs = 0b1011001110001101
    qg = nvq.quant_cols_rht(to_dev(g), signs, sr=True, seed=5)
    qx = nvq.quant_cols_rht(to_dev(x), signs)
    dw = nvq.mm(qg, qx, out_dtype=torch.float32)
    check_close(dw, ref_product(qg, qx, nvq), bf16=False)
    assert rel_fro(dw.cpu().numpy(), g.astype(np.float64).T @ x.astype(np.float64)) < 0.2
    L.check_status()


def test_gemm_rejects_bad_arguments(mods):
    nvq, _, L = mods
    lib = L.load()
    t = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    c = torch.zeros(128, 128, device="cuda")
    p, st = t.data_ptr(), L.stream()
    args = lambda **kw: [kw.get("a", p), p, kw.get("lda", 64), p, p, 64, c.data_ptr(), kw.get("cd", 1), 128,
                         kw.get("M", 128), 128, kw.get("K", 128), 0, None, None, 1.0, 1.0, kw.get("acc", 0), 1, None, st]
    assert lib.nvfp4_gemm(*args()) == 0
    assert lib.nvfp4_gemm(*args(M=100)) == -2
    assert lib.nvfp4_gemm(*args(K=96)) == -2
    assert lib.nvfp4_gemm(*args(lda=72)) == -3
    assert lib.nvfp4_gemm(*args(a=p + 8)) == -3
    assert lib.nvfp4_gemm(*args(a=None)) == -1
    assert lib.nvfp4_gemm(*args(cd=0, acc=1)) == -4
    torch.cuda.synchronize()


@pytest.mark.parametrize("M,N,K,owners,splitk", [(1024, 512, 4096, 4, 1), (512, 384, 2048, 2, 1), (2048, 256, 8192, 8, 0),
                                                  (256, 256, 1024, 1, 1)])
def test_scatter_rows_adds_each_row_slab_into_its_owner(mods, M, N, K, owners, splitk):
    """The weight-gradient GEMM with the reduce-scatter in its epilogue, on one GPU: every "rank's" copy of C is a
    buffer of its own here.  Owner r receives product + what it held in rows [r M / n, (r + 1) M / n) and nothing
    anywhere else; with one K slice the sums are bit-equal to the accumulating GEMM's."""
    nvq, _, L = mods
    qa = nvq.quant_rows(to_dev(make_x(M + 1, M, K)))
    qb = nvq.quant_rows(to_dev(make_w(N + 2, N, K)))
    want = torch.full((M, N), 0.5, device="cuda")
    nvq.mm(qa, qb, out_dtype=torch.float32, out=want, accumulate=True, splitk=1)
    bufs = [torch.full((M, N), 0.5, device="cuda") for _ in range(owners)]
    nvq.mm(qa, qb, out_dtype=torch.float32, out=bufs[0], splitk=splitk, owners=[b.data_ptr() for b in bufs])
    torch.cuda.synchronize()
    L.check_status()
    rows = M // owners
    for r, b in enumerate(bufs):
        mine = slice(r * rows, (r + 1) * rows)
        if splitk == 1:
            assert torch.equal(b[mine], want[mine]), r
        else:
            check_close(b[mine], want[mine].double().cpu().numpy(), bf16=False)
        rest = torch.cat([b[:r * rows], b[(r + 1) * rows:]])
        assert bool((rest == 0.5).all()), r


def test_scatter_rows_rejects_bad_requests(mods):
    nvq, _, L = mods
    lib = L.load()
    M, N, K = 768, 256, 1024
    qa = nvq.quant_rows(to_dev(make_x(1, M, K)))
    qb = nvq.quant_rows(to_dev(make_w(2, N, K)))
    out = torch.zeros(M, N, device="cuda")

    def call(ptrs, m=M):
        return lib.nvfp4_gemm_scatter_rows(L.ptr(qa.d), L.ptr(qa.s), qa.d.stride(0), L.ptr(qb.d), L.ptr(qb.s), qb.d.stride(0),
                                           L.ptr_array(ptrs) if ptrs is not None else None, len(ptrs or []), N, m, N, K,
                                           L.ALPHA_GS, L.ptr(qa.gs), L.ptr(qb.gs), 1.0, 1.0, 1, None, L.stream())
    p = out.data_ptr()
    assert call(None) == -1                      # null
    assert call([p] * 4) == -2                   # shape: 768 / 4 = 192 rows per owner are not whole 128-row tiles
    assert call([p] * 9) == -2
    assert call([p, 0, p]) == -1
    assert call([p, p + 4, p]) == -3              # alignment
    assert call([p] * 3) == 0                    # 256 rows each
    torch.cuda.synchronize()
    L.check_status()
