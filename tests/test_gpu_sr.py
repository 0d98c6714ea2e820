"""Hardware stochastic rounding (cvt.rs.satfinite.e2m1x4.f32): the CPU model reproduces the
instruction bit-for-bit on identical random bits, the quantizers built on it match the oracle,
and the rounding is unbiased within stated bounds."""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from tests.gpu_util import make_dy, to_dev, u8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L():
    from nvfp4_training_b200 import _lib
    _lib.load()
    return _lib


def hw_convert(L, y, words):
    yt = torch.from_numpy(np.ascontiguousarray(y, dtype=np.float32)).cuda()
    wt = torch.from_numpy(np.ascontiguousarray(words, dtype=np.uint32).view(np.int32)).cuda()
    out = torch.empty(words.size, dtype=torch.int16, device="cuda")
    L.check(L.load().nvfp4_e2m1x4_sr(yt.data_ptr(), wt.data_ptr(), out.data_ptr(), words.size, L.stream()), "sr")
    return out.cpu().numpy().view(np.uint16)


def model_convert(y, words):
    lanes = O.hw_lane_bits(words)                                   # [n, 4]
    codes = O.sr_hw_code(y.reshape(-1, 4), lanes).astype(np.uint16)
    return codes[:, 0] | (codes[:, 1] << 4) | (codes[:, 2] << 8) | (codes[:, 3] << 12)


def test_cvt_rs_model_bit_exact(L):
    rng = np.random.default_rng(0)
    n = 1 << 18
    y = np.concatenate([
        rng.uniform(-6.5, 6.5, 2 * n), rng.standard_normal(n) * 2, rng.uniform(-1, 1, n) * 0.6,
        (rng.integers(-28, 29, n) * 0.25), np.array([0.0, -0.0, 6.0, -6.0, 1e-30, -1e-30, 1e30, np.inf, -np.inf, 7.0, 5.9999995, 0.25]),
    ]).astype(np.float32)
    y = y[: (y.size // 4) * 4]
    words = rng.integers(0, 1 << 32, y.size // 4, dtype=np.uint64).astype(np.uint32)
    assert np.array_equal(hw_convert(L, y, words), model_convert(y, words))
    # extremes of the random word
    for w in (0, 0xFFFFFFFF, 0x00FF00FF, 0xFF00FF00, 0x0000FFFF):
        ww = np.full(y.size // 4, w, dtype=np.uint32)
        assert np.array_equal(hw_convert(L, y, ww), model_convert(y, ww))


def test_cvt_rs_unbiased_per_value(L):
    """Stated bound: for each v on a 1024-point grid in [0, 6] and n = 2^14 draws with uniformly
    random words (all four lanes of the instruction take part),
    |mean - v| <= 5 * step(v) * sqrt(p(1-p)/n) + step(v) * 2^-16, p the fractional position of v."""
    rng = np.random.default_rng(1)
    grid = np.linspace(0, 6, 1024, dtype=np.float32)
    n = 1 << 14
    y4 = np.repeat(grid, n)
    words = rng.integers(0, 1 << 32, y4.size // 4, dtype=np.uint64).astype(np.uint32)
    packed = hw_convert(L, y4, words)
    tab = O.E2M1_TABLE.astype(np.float64)
    vals = sum(tab[(packed >> (4 * j)) & 15] for j in range(4)) / 4.0
    mean = vals.reshape(grid.size, -1).mean(1)
    step = np.where(grid < 2, 0.5, np.where(grid < 4, 1.0, 2.0))
    lo = np.floor(grid / step) * step
    p = (grid - lo) / step
    bound = 5 * step * np.sqrt(p * (1 - p) / n) + step * 2.0 ** -16 + 1e-9
    assert np.all(np.abs(mean - grid) <= bound), float(np.max(np.abs(mean - grid) / bound))


@pytest.mark.parametrize("seed", [0, 123456789])
def test_quantizers_hw_sr_bit_exact(L, seed):
    from nvfp4_training_b200 import nvq
    old = nvq.SR_MODE
    nvq.SR_MODE = L.ROUND_SR_HW
    try:
        x = make_dy(21, 256, 384)
        codes, scales, gs = O.quant_rows(x, sr_mode=O.SR_HW, seed=seed)
        q = nvq.quant_rows(to_dev(x), sr=True, seed=seed)
        assert np.array_equal(u8(q.d), codes)
        assert np.array_equal(O.unswizzle_scales(u8(q.s), 256, 24), scales) and q.gs.item() == float(gs)
        codes, scales, gs = O.quant_cols_rht(x, 0xA5C3, sr_mode=O.SR_HW, seed=seed)
        q = nvq.quant_cols_rht(to_dev(x), 0xA5C3, sr=True, seed=seed)
        assert np.array_equal(u8(q.d), codes)
        assert np.array_equal(O.unswizzle_scales(u8(q.s), 384, 16), scales) and q.gs.item() == float(gs)
    finally:
        nvq.SR_MODE = old


def test_hw_sr_mean_of_64(L):
    from nvfp4_training_b200 import nvq
    old = nvq.SR_MODE
    nvq.SR_MODE = L.ROUND_SR_HW
    try:
        x = to_dev(make_dy(9, 512, 384))
        xf = x.float()
        acc = torch.zeros_like(xf)
        for s in range(64):
            acc += nvq.dequant(nvq.quant_rows(x, sr=True, seed=s))
        e_sr = ((acc / 64 - xf).norm() / xf.norm()).item()
        e_rn = ((nvq.dequant(nvq.quant_rows(x)) - xf).norm() / xf.norm()).item()
        assert e_sr <= 0.25 * e_rn, (e_sr, e_rn)
    finally:
        nvq.SR_MODE = old
