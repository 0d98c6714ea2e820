"""GPU parity at the shapes the benchmark configurations name (seeded synthetic inputs with their
distributions: X ~ N(0,1) with 8 outlier columns x30, W ~ N(0, 0.02), dY ~ Student-t(3) * 1e-3).

  config 1   X [4096, 2048] rows 1x16, W [2048, 2048] 16x16 blocks, round to nearest: codes, scale bytes and
             gs bit-exact against the oracle, Y = deq(X) deq(W)^T against the FP64 product of the dequantized
             operands (whole matrix).
  config 2   every projection of one 1B block at T = 4096 -- qkv 2048->3072, o 3072->2048 and the
             reference's 2048->2048, gate/up 2048->11264, down 5632->2048 -- fprop, dgrad and wgrad through
             the quantizers of the layer recipe; each GEMM against the FP64 product of the bytes it was given
             on 8 sampled rows of every 128-row block (all tiles are hit), round-to-nearest operands bit-exact
             against the oracle, stochastic ones on row / column bands.
  config 3   wgrad stress: dY [16384, 5632] stochastic, X [16384, 2048] nearest, RHT16 on both, FP32 dW
             [5632, 2048]: sampled rows against FP64, and the relative error against the exact dY^T X.

GEMM tolerances (every product is exact in FP32; only the accumulation order differs):
  FP32 output  |C - Y| <= 1e-4 |Y| + 1e-6 max|Y|  and  ||C - Y||_F <= 1e-5 ||Y||_F
  bf16 output  |C - Y| <= 2^-8 |Y| + 1e-6 max|Y|  and  ||C - Y||_F <= 4e-3 ||Y||_F
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
    from nvfp4_training_b200 import _lib, nvq
    _lib.load()
    yield nvq, _lib
    _lib.check_status()


def sample_rows(R, per_block=8, seed=0):
    rng = np.random.default_rng(seed)
    return np.concatenate([b * 128 + np.sort(rng.choice(128, per_block, replace=False)) for b in range(R // 128)])


def deq_rows(q, rows=None):
    """float64 [len(rows), C] block-scaled values (without the tensor scale) of the rows of a packed operand."""
    R, C = q.d.shape[0], q.d.shape[1] * 2
    codes = u8(q.d)
    scales = O.unswizzle_scales(u8(q.s), R, C // 16)
    if rows is not None:
        codes, scales = codes[rows], scales[rows]
    return (O.E2M1_TABLE[O.unpack_codes(codes)] * np.repeat(O.e4m3_decode(scales), 16, axis=1)).astype(np.float64)


def check_gemm_rows(c, qa, qb, rows, bf16):
    """C[rows] against the FP64 product of the dequantized operand bytes."""
    y = deq_rows(qa, rows) @ deq_rows(qb).T * (float(qa.gs.item()) * float(qb.gs.item()))
    got = c[torch.from_numpy(rows).cuda()].float().cpu().numpy().astype(np.float64)
    fro, rel = (4e-3, 2.0 ** -8) if bf16 else (1e-5, 1e-4)
    assert rel_fro(got, y) <= fro, rel_fro(got, y)
    bad = np.abs(got - y) > rel * np.abs(y) + 1e-6 * np.abs(y).max()
    assert not bad.any(), (int(bad.sum()), float(np.abs(got - y).max()))


def check_q(q, codes, scales, gs, rows=None):
    R, C = q.d.shape[0], q.d.shape[1] * 2
    got_c, got_s = u8(q.d), O.unswizzle_scales(u8(q.s), R, C // 16)
    if rows is not None:
        got_c, got_s = got_c[rows], got_s[rows]
    assert np.array_equal(got_c, codes) and np.array_equal(got_s, scales)
    assert q.gs.item() == float(gs)


def test_config1_roundtrip_and_gemm(mods):
    nvq, L = mods
    x, w = make_x(0, 4096, 2048, outliers=8), make_w(0, 2048, 2048)
    qx = nvq.quant_rows(to_dev(x))
    qw, qwt = nvq.quant_w2d(to_dev(w))
    check_q(qx, *O.quant_rows(x))
    oq, os_, oqt, ost, ogs = O.quant_w2d(w)
    check_q(qw, oq, os_, ogs)
    check_q(qwt, oqt, ost, ogs)
    rows = np.arange(4096)
    check_gemm_rows(nvq.mm(qx, qw, out_dtype=torch.float32), qx, qw, rows, bf16=False)
    check_gemm_rows(nvq.mm(qx, qw), qx, qw, rows, bf16=True)
    # the reference's own check (llm-1b/test_nvq.py:12): FP32 matmul of the torch-decoded operands
    y = nvq.dequant(qx) @ nvq.dequant(qw).t()
    assert ((nvq.mm(qx, qw, out_dtype=torch.float32) - y).norm() / y.norm()).item() < 1e-5
    L.check_status()


PROJECTIONS = [("qkv", 3072, 2048), ("o_baseline", 2048, 3072), ("o_reference", 2048, 2048),
               ("gate_up", 11264, 2048), ("down", 2048, 5632)]


@pytest.mark.parametrize("name,N,K", PROJECTIONS)
def test_config2_projection_fprop_dgrad_wgrad(mods, name, N, K):
    nvq, L = mods
    T = 4096
    x, w, gy = make_x(1, T, K, outliers=0), make_w(2, N, K), make_dy(3, T, N)
    xd, gyd = to_dev(x), to_dev(gy)
    qw, qwt = nvq.quant_w2d(to_dev(w))
    am_x, am_g = nvq.amax(xd), nvq.amax(gyd)
    ax, ag = O.amax_f32(x), O.amax_f32(gy)
    assert am_x.item() == float(ax) and am_g.item() == float(ag)
    # forward: both operands of x from one pass (round to nearest): whole-tensor byte equality
    qx, qxt = nvq.quant_rows_cols_rht(xd, SIGNS, am=am_x)
    check_q(qx, *O.quant_rows(x, amax=ax))
    check_q(qxt, *O.quant_cols_rht(x, SIGNS, amax=ax))
    y = nvq.mm(qx, qw)
    check_gemm_rows(y, qx, qw, sample_rows(T, seed=1), bf16=True)
    # backward: both operands of gy, stochastic (the reference's dither rounding and stream), checked on bands
    seed = (5 * 1000003 + 11 * 7919) & 0xFFFFFFFF
    qg, qgt = nvq.quant_rows_cols_rht(gyd, SIGNS, sr=True, seed=seed, seed_cols=seed ^ 0x5BD1E995, am=am_g)
    for r0 in (0, T // 2 + 128, T - 128):
        rows = np.arange(r0, r0 + 128)
        check_q(qg, *O.quant_rows(gy[rows], amax=ag, sr_mode=O.SR_DITHER_NVQ, seed=seed, blk0=r0 * (N // 16)), rows=rows)
    for c0 in (0, N // 2 + 64, N - 64):
        cols = np.arange(c0, c0 + 64)
        check_q(qgt, *O.quant_cols_rht(gy[:, cols], SIGNS, amax=ag, sr_mode=O.SR_DITHER_NVQ, seed=seed ^ 0x5BD1E995,
                                       blk0=c0 * (T // 16)), rows=cols)
    gx = nvq.mm(qg, qwt)
    check_gemm_rows(gx, qg, qwt, sample_rows(T, seed=2), bf16=True)
    gw = nvq.mm(qgt, qxt, out_dtype=torch.float32)
    check_gemm_rows(gw, qgt, qxt, sample_rows(N, seed=3), bf16=False)
    # accumulate a second microbatch in place (first call overwrites, second adds)
    gw2 = torch.empty_like(gw)
    nvq.mm(qgt, qxt, out_dtype=torch.float32, out=gw2)
    nvq.mm(qgt, qxt, out_dtype=torch.float32, out=gw2, accumulate=True)
    assert torch.equal(gw2, 2 * gw)
    # and the quantized layer tracks the exact one within FP4 noise (llm-1b/test_nvq.py:14-18 bound)
    exact = gyd.double().t() @ xd.double()
    assert ((gw.double() - exact).norm() / exact.norm()).item() < 0.2
    L.check_status()


def test_config3_wgrad_stress(mods):
    nvq, L = mods
    T, N, K = 16384, 5632, 2048
    gy, x = make_dy(7, T, N), make_x(8, T, K, outliers=0)
    gyd, xd = to_dev(gy), to_dev(x)
    rng = np.random.default_rng(0)
    signs = int(rng.integers(0, 1 << 16))
    ag, ax = O.amax_f32(gy), O.amax_f32(x)
    qgt = nvq.quant_cols_rht(gyd, signs, sr=True, seed=9)
    qxt = nvq.quant_cols_rht(xd, signs)
    # X operand: round to nearest, whole tensor; dY operand: stochastic, three column bands
    check_q(qxt, *O.quant_cols_rht(x, signs, amax=ax))
    for c0 in (0, 2816, N - 64):
        cols = np.arange(c0, c0 + 64)
        check_q(qgt, *O.quant_cols_rht(gy[:, cols], signs, amax=ag, sr_mode=O.SR_DITHER_NVQ, seed=9, blk0=c0 * (T // 16)),
                rows=cols)
    dw = nvq.mm(qgt, qxt, out_dtype=torch.float32)
    assert dw.shape == (N, K) and dw.dtype == torch.float32
    check_gemm_rows(dw, qgt, qxt, sample_rows(N, per_block=4, seed=4), bf16=False)
    exact = gyd.double().t() @ xd.double()
    err = ((dw.double() - exact).norm() / exact.norm()).item()
    assert err < 0.2, err
    L.check_status()
