"""GPU parity in the regime the benchmark runs: every persistent / grid-stride loop of the library walks
MANY work items per CTA, so the state carried from one item to the next (stage rings and their phase
bits, accumulator ping-pong, the 48 tensor-memory columns two 256-wide accumulators share, the banded
tile walk, the in-loop drain of the previous tile's transposed outputs) is compared with the oracle.

  * GEMM with `nvfp4_gemm_set_sm_budget(2)` / `(4)`: one or two SM pairs walk dozens of tiles, with more
    than 8 tile columns so the band walk crosses a band and ends in a partial one; every tile variant,
    bf16 / FP32 / accumulate / split-K.  Tolerances as in test_gpu_gemm.py.
  * tile quantizer on 2048 tiles (about 7 per CTA): all four rounding modes, both scale layouts,
    whole-tensor byte equality for round-to-nearest, row / column bands for the stochastic modes.
  * row quantizer on >= 65 536 items and weight quantizer on >= 16 384 items: byte equality.
"""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from tests.gpu_util import make_dy, make_w, make_x, rel_fro, to_dev, u8

pytestmark = pytest.mark.gpu

SIGNS = 0b1010011010110001


@pytest.fixture(scope="module")
def mods():
    from nvfp4_training_b200 import _lib, fp4ops, nvq
    _lib.load()
    yield nvq, fp4ops, _lib
    _lib.load().nvfp4_gemm_force_tile_n(0)
    _lib.load().nvfp4_gemm_set_sm_budget(0)
    _lib.check_status()


_REF = {}


def operands_and_ref(nvq, M, N, K):
    """Quantized operands (cached per shape) and the FP64 product of their dequantized bytes."""
    key = (M, N, K)
    if key not in _REF:
        qa = nvq.quant_rows(to_dev(make_x(M + K, M, K)))
        qb = nvq.quant_rows(to_dev(make_w(N, N, K)))
        sa = O.unswizzle_scales(u8(qa.s), M, K // 16)
        sb = O.unswizzle_scales(u8(qb.s), N, K // 16)
        y = O.gemm_unit(u8(qa.d), sa, u8(qb.d), sb) * (float(qa.gs.item()) * float(qb.gs.item()))
        _REF[key] = (qa, qb, y)
    return _REF[key]


def check_close(c, y, bf16):
    c = c.float().cpu().numpy().astype(np.float64)
    fro, rel = (4e-3, 2.0 ** -8) if bf16 else (1e-5, 1e-4)
    assert rel_fro(c, y) <= fro, rel_fro(c, y)
    bad = np.abs(c - y) > rel * np.abs(y) + 1e-6 * np.abs(y).max()
    assert not bad.any(), (int(bad.sum()), float(np.abs(c - y).max()))


def raw_gemm(L, qa, qb, out, accumulate, splitk):
    M, N, K = qa.d.shape[0], qb.d.shape[0], qa.d.shape[1] * 2
    L.check(L.load().nvfp4_gemm(qa.d.data_ptr(), qa.s.data_ptr(), qa.d.stride(0), qb.d.data_ptr(), qb.s.data_ptr(),
                                qb.d.stride(0), out.data_ptr(), L.DTYPE_FP32 if out.dtype == torch.float32 else L.DTYPE_BF16,
                                out.stride(0), M, N, K, L.ALPHA_GS, qa.gs.data_ptr(), qb.gs.data_ptr(), 1.0, 1.0,
                                int(accumulate), splitk, L.status_word(out.device).data_ptr(), L.stream()), "gemm")
    return out


# N = 2816: 11 tile columns at 256, 15 (the last clipped) at 192, 22 at 128
@pytest.mark.parametrize("budget", [2, 4])
@pytest.mark.parametrize("tile", [0, 128, 256, 512, 448, 384])
@pytest.mark.parametrize("M,N,K", [(512, 2816, 576), (1024, 2816, 2304)])
def test_gemm_many_tiles_per_cta(mods, M, N, K, tile, budget):
    nvq, _, L = mods
    lib = L.load()
    qa, qb, y = operands_and_ref(nvq, M, N, K)
    lib.nvfp4_gemm_force_tile_n(tile)
    assert lib.nvfp4_gemm_set_sm_budget(budget) == 0
    try:
        check_close(nvq.mm(qa, qb), y, bf16=True)
        check_close(nvq.mm(qa, qb, out_dtype=torch.float32), y, bf16=False)
        out = torch.full((M, N), 0.5, device="cuda")
        nvq.mm(qa, qb, out_dtype=torch.float32, out=out, accumulate=True)
        nvq.mm(qa, qb, out_dtype=torch.float32, out=out, accumulate=True)
        check_close(out, 2 * y + 0.5, bf16=False)
        for splitk in (2, 3):
            check_close(raw_gemm(L, qa, qb, torch.zeros(M, N, device="cuda"), 0, splitk), y, bf16=False)
        torch.cuda.synchronize()
    finally:
        lib.nvfp4_gemm_set_sm_budget(0)
        lib.nvfp4_gemm_force_tile_n(0)
    L.check_status()


def test_gemm_full_grid_more_tiles_than_ctas(mods):
    """The whole GPU, default variant choice, a shape with several tiles per SM pair and a ragged last wave:
    1024 x 11264 x 1024 has 176 pair tiles at 256 columns (74 clusters) and 236 at 192."""
    nvq, _, L = mods
    qa, qb, y = operands_and_ref(nvq, 1024, 11264, 1024)
    for tile in (0, 512, 448, 384, 256, 128):
        L.load().nvfp4_gemm_force_tile_n(tile)
        check_close(nvq.mm(qa, qb), y, bf16=True)
        check_close(nvq.mm(qa, qb, out_dtype=torch.float32), y, bf16=False)
    L.load().nvfp4_gemm_force_tile_n(0)
    L.check_status()


# ---------------------------------------------------------------------------------------- quantizers
def _bands(n, width, count):
    """`count` bands of `width` spread over [0, n): first, last and evenly spaced ones."""
    starts = sorted({int(round(i * (n - width) / (count - 1) / width)) * width for i in range(count)})
    return [(s, s + width) for s in starts]


MODES = [("rn", "SR_NONE", "ROUND_NEAREST"), ("dither", "SR_DITHER_NVQ", "ROUND_SR_DITHER"),
         ("dither_k", "SR_DITHER_FP4K", "ROUND_SR_DITHER_K"), ("hw", "SR_HW", "ROUND_SR_HW")]


@pytest.mark.parametrize("path", [0, 1], ids=["tensor_core_fed", "scalar"])
@pytest.mark.parametrize("linear", [False, True])
@pytest.mark.parametrize("name,omode,lmode", MODES)
def test_tile_quantizer_many_tiles_per_cta(mods, name, omode, lmode, linear, path):
    """[8192, 2048]: 2048 tiles of 128 x 64 (scalar kernel) or 1024 of 128 x 128 (tensor-core-fed kernel)
    over 296 CTAs, so the stage ring wraps, the tensor-memory hand-off repeats and the scalar kernel drains
    transposed outputs inside its loop.  Whole-tensor byte equality for round-to-nearest; for the
    stochastic modes 8 row bands (row operand) and 8 column bands (transposed operand), first and last
    included, against the oracle with the bands' block indices."""
    nvq, _, L = mods
    M, C = 8192, 2048
    x = make_dy(21, M, C) if name != "rn" else make_x(22, M, C)
    xd = to_dev(x)
    am = nvq.amax(xd)
    amax = O.amax_f32(x)
    assert am.item() == float(amax)
    dr = torch.empty(M, C // 2, dtype=torch.uint8, device="cuda")
    sr = torch.empty(M * C // 16, dtype=torch.uint8, device="cuda")
    dc = torch.empty(C, M // 2, dtype=torch.uint8, device="cuda")
    sc = torch.empty(C * M // 16, dtype=torch.uint8, device="cuda")
    gr, gc = torch.empty(1, device="cuda"), torch.empty(1, device="cuda")
    seed_r, seed_c = 0x1234567, 0x89ABCDE
    assert L.load().nvfp4_quant_tile_set_path(path) == 0
    try:
        L.check(L.load().nvfp4_quant_tile(xd.data_ptr(), C, M, C, dr.data_ptr(), sr.data_ptr(), dc.data_ptr(), sc.data_ptr(),
                                          L.SCALES_LINEAR if linear else L.SCALES_SWIZZLED, am.data_ptr(), gr.data_ptr(),
                                          gc.data_ptr(), SIGNS, getattr(L, lmode), seed_r, seed_c, None, None, L.stream()), "tile")
    finally:
        L.load().nvfp4_quant_tile_set_path(0)
    torch.cuda.synchronize()
    L.check_status()
    codes_r, codes_c = u8(dr), u8(dc)
    scales_r = u8(sr).reshape(M, C // 16) if linear else O.unswizzle_scales(u8(sr), M, C // 16)
    scales_c = u8(sc).reshape(C, M // 16) if linear else O.unswizzle_scales(u8(sc), C, M // 16)
    om = getattr(O, omode)
    if name == "rn":
        c, s, g = O.quant_rows(x, amax=amax)
        assert np.array_equal(codes_r, c) and np.array_equal(scales_r, s) and gr.item() == float(g)
        c, s, g = O.quant_cols_rht(x, SIGNS, amax=amax)
        assert np.array_equal(codes_c, c) and np.array_equal(scales_c, s) and gc.item() == float(g)
        return
    for r0, r1 in _bands(M, 128, 8):
        c, s, g = O.quant_rows(x[r0:r1], amax=amax, sr_mode=om, seed=seed_r, blk0=r0 * (C // 16))
        assert np.array_equal(codes_r[r0:r1], c) and np.array_equal(scales_r[r0:r1], s), (r0, r1)
        assert gr.item() == float(g)
    for c0, c1 in _bands(C, 64, 8):
        c, s, g = O.quant_cols_rht(x[:, c0:c1], SIGNS, amax=amax, sr_mode=om, seed=seed_c, blk0=c0 * (M // 16))
        assert np.array_equal(codes_c[c0:c1], c) and np.array_equal(scales_c[c0:c1], s), (c0, c1)
        assert gc.item() == float(g)


@pytest.mark.parametrize("R,C", [(66048, 64), (16384, 2048)])
def test_quant_rows_many_items_per_warp(mods, R, C):
    """The row kernel walks (row, 512-column segment) items with a fixed warp stride: 66 048 and 65 536
    items against at most 18 944 warps, so every warp takes several items and prefetches across them."""
    nvq, fp4ops, _ = mods
    x = make_x(31, R, C, outliers=4)
    codes, scales, gs = O.quant_rows(x)
    q = nvq.quant_rows(to_dev(x))
    assert np.array_equal(u8(q.d), codes)
    assert np.array_equal(O.unswizzle_scales(u8(q.s), R, C // 16), scales)
    assert q.gs.item() == float(gs)
    if C == 64:
        # the fp4ops flavour (mantissa dither, element-indexed stream, linear scales) on the last row band
        c, s, _ = O.quant_rows(x[-256:], amax=O.amax_f32(x), sr_mode=O.SR_DITHER_FP4K, seed=5, blk0=(R - 256) * (C // 16))
        qf = fp4ops.quant_rows(to_dev(x), sr=True, seed=5)
        assert np.array_equal(u8(qf.d)[-256:], c) and np.array_equal(u8(qf.s)[-256:], s)


def test_quant_w2d_many_items_per_warp(mods):
    """[11264, 2048]: 176 x 128 = 22 528 warp items (groups of four 16x16 blocks) against 9 472 warps."""
    nvq, _, _ = mods
    N, K = 11264, 2048
    w = make_w(41, N, K)
    q, s, qt, st, gs = O.quant_w2d(w)
    a, b = nvq.quant_w2d(to_dev(w))
    assert np.array_equal(u8(a.d), q) and np.array_equal(O.unswizzle_scales(u8(a.s), N, K // 16), s)
    assert np.array_equal(u8(b.d), qt) and np.array_equal(O.unswizzle_scales(u8(b.s), K, N // 16), st)
    assert a.gs.item() == float(gs)


def test_cols_rht_fallback_kernel_large(mods):
    """The register-tiled column kernel (shapes the tile kernel does not take: M % 128 != 0) on a grid of
    many CTAs in both dimensions."""
    nvq, _, _ = mods
    M, C = 4160, 1024                      # M % 128 == 64
    x = make_dy(51, M, C)
    codes, scales, gs = O.quant_cols_rht(x, SIGNS)
    q = nvq.quant_cols_rht(to_dev(x), SIGNS)
    assert np.array_equal(u8(q.d), codes)
    assert np.array_equal(O.unswizzle_scales(u8(q.s), C, M // 16), scales)
    assert q.gs.item() == float(gs)


def test_gemm_items_dealt_in_advance_equal_drawn_at_run_time():
    """The CTA-pair kernel with its work items drawn at run time (default) and dealt out in advance: same bytes out
    (every item is computed once, by whichever cluster takes it), under an SM budget that makes every cluster walk
    many items, for bf16, FP32 and accumulating outputs."""
    from nvfp4_training_b200 import _lib as L, nvq
    lib = L.load()
    M, N, K = 1024, 2816, 2304
    qa = nvq.quant_rows(to_dev(make_x(1, M, K)))
    qb = nvq.quant_rows(to_dev(make_w(2, N, K)))
    outs = {}
    try:
        for mode in (1, 2, 0):
            assert lib.nvfp4_gemm_set_scheduler(mode) == 0
            for budget in (0, 4):
                lib.nvfp4_gemm_set_sm_budget(budget)
                y16 = nvq.mm(qa, qb)
                y32 = nvq.mm(qa, qb, out_dtype=torch.float32)
                acc = torch.ones(M, N, device="cuda")
                nvq.mm(qa, qb, out_dtype=torch.float32, out=acc, accumulate=True)
                outs[(mode, budget)] = (y16, y32, acc)
    finally:
        lib.nvfp4_gemm_set_scheduler(1)
        lib.nvfp4_gemm_set_sm_budget(0)
    L.check_status()
    ref = outs[(0, 0)]
    for key, got in outs.items():
        for a, b in zip(ref, got):
            assert torch.equal(a, b), key
    assert ref[1].abs().max().item() > 0
