"""GPU parity of the quantizer kernels against the CPU oracle: codes, scale bytes and tensor scales
bit-exact for round-to-nearest and for stochastic rounding given the same random bits."""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from tests.gpu_util import bf16_round, make_dy, make_w, make_x, to_dev, u8

pytestmark = pytest.mark.gpu

ROW_CASES = ["normal_outliers", "weights_small", "student_t", "ties", "range", "zeros", "tiny", "negzero"]


@pytest.fixture(scope="module")
def mods():
    from nvfp4_training_b200 import _lib, fp4ops, nvq
    _lib.load()
    return nvq, fp4ops, _lib


def check_nvq(q, codes, scales, gs, R, C):
    assert np.array_equal(u8(q.d), codes)
    assert np.array_equal(O.unswizzle_scales(u8(q.s), R, C // 16), scales)
    assert q.gs.item() == float(gs)


def test_amax(mods):
    nvq, _, _ = mods
    for n, seed in [(8, 0), (4096, 1), (128 * 2048, 2), (1 << 22, 3), ((1 << 22) + 8 * 77, 4)]:
        rng = np.random.default_rng(seed)
        x = bf16_round(rng.standard_normal(n).astype(np.float32) * 3)
        x[rng.integers(n)] = -77.5
        assert nvq.amax(to_dev(x)).item() == float(O.amax_f32(x))
    assert nvq.amax(torch.zeros(64, dtype=torch.bfloat16, device="cuda")).item() == 0.0
    out = torch.full((1,), 9.0, device="cuda")
    nvq.amax(to_dev(np.full(16, 0.5, dtype=np.float32)), out=out)
    assert out.item() == 0.5


@pytest.mark.parametrize("name", ROW_CASES)
def test_rows_rn_golden_inputs(mods, golden, name):
    nvq, fp4ops, _ = mods
    x = O.bf16_bits_to_f32(golden[f"rows_{name}_x"])
    R, C = x.shape
    codes, scales, gs = O.quant_rows(x)
    q = nvq.quant_rows(to_dev(x))
    check_nvq(q, codes, scales, gs, R, C)
    # dequantized result equals the reference's torch fake-quant, bit for bit
    assert np.array_equal(nvq.dequant(q).cpu().numpy(), golden[f"rows_{name}_dq"])
    # linear-scale flavour
    qf = fp4ops.quant_rows(to_dev(x))
    assert np.array_equal(u8(qf.d), codes) and np.array_equal(u8(qf.s), scales)
    assert np.array_equal(fp4ops.dequant(qf).cpu().numpy(), golden[f"rows_{name}_dq"])


@pytest.mark.parametrize("R,C,seed", [(128, 64, 0), (256, 576, 1), (4096, 2048, 0), (384, 5632, 2)])
def test_rows_rn_shapes(mods, R, C, seed):
    nvq, _, _ = mods
    x = make_x(seed, R, C)
    codes, scales, gs = O.quant_rows(x)
    check_nvq(nvq.quant_rows(to_dev(x)), codes, scales, gs, R, C)


def test_rows_strided_and_shared_amax(mods):
    nvq, _, _ = mods
    x = make_dy(5, 256, 512)
    big = to_dev(np.concatenate([x, x], axis=1))
    view = big[:, 512:]                       # row stride 1024, offset 512
    am = nvq.amax(to_dev(x))
    am4 = am * 4
    codes, scales, gs = O.quant_rows(x, amax=O.amax_f32(x) * np.float32(4))
    check_nvq(nvq.quant_rows(view, am=am4), codes, scales, gs, 256, 512)


@pytest.mark.parametrize("top", [48.0, 2688.0])
def test_rows_fast_path_boundaries(mods, top):
    """Values whose scaled magnitude sits exactly on, or one bf16 step around, every rounding
    boundary of the E2M1 grid: the FMA divisions must round exactly like IEEE divisions."""
    nvq, _, _ = mods
    rng = np.random.default_rng(11)
    bounds = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    x = np.zeros((128, 64), dtype=np.float32)
    for r in range(128):
        for b in range(4):
            blk = rng.choice(bounds, 16) * rng.choice([-1.0, 1.0], 16)
            blk[rng.integers(16)] = 6.0                      # block max -> scale exactly 2^k
            x[r, b * 16:(b + 1) * 16] = blk * 2.0 ** rng.integers(-3, 4)
    x[0, 0] = top          # tensor amax: 2688 makes gs = 1, so every scaled value is an exact tie
    x = bf16_round(x)
    codes, scales, gs = O.quant_rows(x)
    check_nvq(nvq.quant_rows(to_dev(x)), codes, scales, gs, 128, 64)


def test_rows_signed_zeros_and_tiny_values(mods):
    """-0 and values far below the block scale keep their sign in the code (0x8 for negative zero)."""
    nvq, _, _ = mods
    rng = np.random.default_rng(4)
    x = rng.standard_normal((128, 128)).astype(np.float32)
    x[:, ::3] = -0.0
    x[:, 1::5] = 0.0
    x[:, 2::7] = -1e-30
    x[:, 4::11] = 1e-38
    x[5, :16] = -0.0                     # a whole block of negative zeros (scale byte 0)
    x = bf16_round(x)
    codes, scales, gs = O.quant_rows(x)
    check_nvq(nvq.quant_rows(to_dev(x)), codes, scales, gs, 128, 128)


def test_rows_16_byte_aligned_rows(mods):
    """Rows that are 16- but not 32-byte aligned take the 128-bit load variant."""
    nvq, _, _ = mods
    x = make_x(9, 128, 256)
    big = to_dev(np.concatenate([np.zeros((128, 8), np.float32), x], axis=1))   # row stride 264
    view = big[:, 8:]
    codes, scales, gs = O.quant_rows(x)
    check_nvq(nvq.quant_rows(view), codes, scales, gs, 128, 256)


@pytest.mark.parametrize("mode_name", ["SR_DITHER_NVQ", "SR_DITHER_FP4K"])
@pytest.mark.parametrize("seed", [0, 7, 0xDEADBEEF])
def test_rows_sr_dither_bit_exact(mods, mode_name, seed):
    nvq, fp4ops, L = mods
    x = make_dy(3, 256, 320 if mode_name == "SR_DITHER_FP4K" else 384)
    R, C = x.shape
    codes, scales, gs = O.quant_rows(x, sr_mode=getattr(O, mode_name), seed=seed)
    if mode_name == "SR_DITHER_NVQ":
        assert nvq.SR_MODE == L.ROUND_SR_DITHER
        check_nvq(nvq.quant_rows(to_dev(x), sr=True, seed=seed), codes, scales, gs, R, C)
    else:
        assert fp4ops.SR_MODE == L.ROUND_SR_DITHER_K
        q = fp4ops.quant_rows(to_dev(x), sr=True, seed=seed)
        assert np.array_equal(u8(q.d), codes) and np.array_equal(u8(q.s), scales)


def test_rows_sr_unbiased_mean_of_64(mods):
    """llm-1b/test_nvq.py:19-22 / small-model/test_fp4ops.py:12-16: the mean of 64 SR
    quantizations is much closer to x than one round-to-nearest quantization.
    Stated bound: rel-err(mean of 64) <= 1/4 rel-err(RN)."""
    nvq, _, _ = mods
    x = to_dev(make_dy(9, 512, 384))
    xf = x.float()
    acc = torch.zeros_like(xf)
    for s in range(64):
        acc += nvq.dequant(nvq.quant_rows(x, sr=True, seed=s))
    e_sr = ((acc / 64 - xf).norm() / xf.norm()).item()
    e_rn = ((nvq.dequant(nvq.quant_rows(x)) - xf).norm() / xf.norm()).item()
    assert e_sr <= 0.25 * e_rn, (e_sr, e_rn)


def test_w2d_bf16(mods, golden):
    nvq, _, _ = mods
    w = O.bf16_bits_to_f32(golden["w2d_bf16_w"])
    wp = np.zeros((128, 256), dtype=np.float32)
    wp[:, :192] = w                                            # swizzled layout wants K % 128 == 0
    q, s, qt, st, gs = O.quant_w2d(wp)
    a, b = nvq.quant_w2d(to_dev(wp))
    check_nvq(a, q, s, gs, 128, 256)
    check_nvq(b, qt, st, gs, 256, 128)
    assert np.array_equal(nvq.dequant(a).cpu().numpy()[:, :192], golden["w2d_bf16_dq"])
    assert (nvq.dequant(b) - nvq.dequant(a).t()).abs().max().item() == 0.0     # llm-1b/test_nvq.py:11
    only_t = nvq.quant_w2d(to_dev(wp), want=(False, True))
    assert only_t[0] is None and np.array_equal(u8(only_t[1].d), qt)


@pytest.mark.parametrize("N,K,seed", [(2048, 2048, 0), (384, 1152, 1)])
def test_w2d_shapes(mods, N, K, seed):
    nvq, _, _ = mods
    w = make_w(seed, N, K)
    q, s, qt, st, gs = O.quant_w2d(w)
    a, b = nvq.quant_w2d(to_dev(w))
    check_nvq(a, q, s, gs, N, K)
    check_nvq(b, qt, st, gs, K, N)


def test_w2d_fp32_linear(mods, golden):
    _, fp4ops, _ = mods
    w = golden["w2d_f32_w"]
    q, s, qt, st, gs = O.quant_w2d(w)
    a, b = fp4ops.quant_w2d(torch.from_numpy(w).cuda())
    assert np.array_equal(u8(a.d), q) and np.array_equal(u8(a.s), s)
    assert np.array_equal(u8(b.d), qt) and np.array_equal(u8(b.s), st)
    assert np.array_equal(fp4ops.dequant(a).cpu().numpy(), golden["w2d_f32_dq"])     # small-model/test_fp4ops.py:18-21
    assert (fp4ops.dequant(b) - fp4ops.dequant(a).t()).abs().max().item() == 0.0


@pytest.mark.parametrize("M,C,seed,kind", [(64, 128, 0, "int"), (256, 384, 1, "t"), (4096, 256, 2, "n"), (16384, 128, 3, "t")])
def test_cols_rht_rn(mods, golden, M, C, seed, kind):
    nvq, fp4ops, _ = mods
    signs = 0b1010011010110001
    if kind == "int":
        x = O.bf16_bits_to_f32(golden["rht_int_x"])
    elif kind == "t":
        x = make_dy(seed, M, C)
    else:
        x = make_x(seed, M, C)
    codes, scales, gs = O.quant_cols_rht(x, signs)
    q = nvq.quant_cols_rht(to_dev(x), signs)
    check_nvq(q, codes, scales, gs, C, M)
    if kind == "int":
        assert np.array_equal(nvq.dequant(q).cpu().numpy(), golden["rht_int_dq"])
    qf = fp4ops.quant_cols_rht(to_dev(x), signs)
    assert np.array_equal(u8(qf.d), codes) and np.array_equal(u8(qf.s), scales) and qf.k == 4.0


@pytest.mark.parametrize("signs", [0, 0xFFFF, 0xA5C3])
def test_cols_rht_sr_dither_bit_exact(mods, signs):
    nvq, fp4ops, _ = mods
    x = make_dy(4, 128, 256)
    am = np.float32(O.amax_f32(x) * np.float32(1.5))
    codes, scales, gs = O.quant_cols_rht(x, signs, amax=am, sr_mode=O.SR_DITHER_NVQ, seed=5)
    amt = torch.tensor([float(am)], device="cuda")
    check_nvq(nvq.quant_cols_rht(to_dev(x), signs, sr=True, seed=5, am=amt), codes, scales, gs, 256, 128)
    codes, scales, gs = O.quant_cols_rht(x, signs, amax=am, sr_mode=O.SR_DITHER_FP4K, seed=5)
    q = fp4ops.quant_cols_rht(to_dev(x), signs, sr=True, seed=5, amax=amt)
    assert np.array_equal(u8(q.d), codes) and np.array_equal(u8(q.s), scales)


SR_MODES = {"rn": None, "dither": "SR_DITHER_NVQ", "dither_k": "SR_DITHER_FP4K", "hw": "SR_HW"}


def codes_equal_up_to_negative_zero(got, want, x_negzero):
    """Packed codes equal except that positions whose INPUT was exactly -0 may carry code 0x0 instead of
    0x8 (the tensor-core-fed kernel's documented difference); magnitudes must agree everywhere."""
    g, w = O.unpack_codes(got), O.unpack_codes(want)
    diff = g != w
    if not diff.any():
        return True
    return bool(np.all(x_negzero[diff]) and np.all((g[diff] & 7) == 0) and np.all((w[diff] & 7) == 0))


@pytest.fixture(params=[0, 1], ids=["tensor_core_fed", "scalar"])
def tile_path(request, mods):
    """Both kernels behind nvfp4_quant_tile: 0 = tensor-core fed where the shape allows, 1 = scalar."""
    lib = mods[2].load()
    assert lib.nvfp4_quant_tile_set_path(request.param) == 0
    yield request.param
    lib.nvfp4_quant_tile_set_path(0)


@pytest.mark.parametrize("mode", ["rn", "dither", "dither_k", "hw"])
@pytest.mark.parametrize("M,C", [(128, 128), (384, 640), (2048, 256)])
def test_tile_quantizer_matches_both_oracles(mods, tile_path, mode, M, C):
    """The one-read tile kernel gives the row operand and the transposed RHT operand bit for bit,
    in every rounding mode, with separate seeds for the two outputs."""
    nvq, _, L = mods
    signs = 0x9C3A
    x = make_dy(M + C, M, C)
    x[5, :16] = 0.0                 # an all-zero block (scale byte 0)
    if tile_path == 1:
        x[16:32, 3] = -0.0          # signed zeros: bit-exact in the scalar kernel (the other kernel: next test)
    xd = to_dev(x)
    if mode == "rn":
        r = O.quant_rows(x)
        c = O.quant_cols_rht(x, signs)
        qr, qc = nvq.quant_rows_cols_rht(xd, signs)
    else:
        om = getattr(O, SR_MODES[mode])
        lm = {"dither": L.ROUND_SR_DITHER, "dither_k": L.ROUND_SR_DITHER_K, "hw": L.ROUND_SR_HW}[mode]
        r = O.quant_rows(x, sr_mode=om, seed=11)
        c = O.quant_cols_rht(x, signs, sr_mode=om, seed=0xBEEF)
        qr, qc = nvq.quant_rows_cols_rht(xd, signs, sr=True, seed=11, seed_cols=0xBEEF, sr_mode=lm)
    check_nvq(qr, r[0], r[1], r[2], M, C)
    check_nvq(qc, c[0], c[1], c[2], C, M)
    assert nvq.quant_tile_status() == 0


def test_tile_quantizer_tensor_core_path_negative_zero_inputs(mods):
    """The tensor-core-fed kernel moves values through an MMA with a 0/1 matrix; an input that is exactly -0
    comes out as +0, so its code may be 0x0 where the convert instruction gives 0x8.  Everything else --
    negative values that round to zero included -- keeps its sign; magnitudes and scales are unchanged."""
    nvq, _, L = mods
    assert L.load().nvfp4_quant_tile_set_path(0) == 0
    M, C, signs = 256, 256, 0x9C3A
    x = make_dy(77, M, C)
    x[16:32, 3] = -0.0
    x[40, 64:80] = -0.0             # a whole row block of negative zeros
    x[:, 200] = -1e-30              # negative and far below every block scale: rounds to -0, sign kept
    x = bf16_round(x)
    negz = (x == 0) & np.signbit(x)
    r = O.quant_rows(x)
    c = O.quant_cols_rht(x, signs)
    qr, qc = nvq.quant_rows_cols_rht(to_dev(x), signs)
    assert np.array_equal(O.unswizzle_scales(u8(qr.s), M, C // 16), r[1]) and qr.gs.item() == float(r[2])
    assert np.array_equal(O.unswizzle_scales(u8(qc.s), C, M // 16), c[1]) and qc.gs.item() == float(c[2])
    assert codes_equal_up_to_negative_zero(u8(qr.d), r[0], negz)
    # transposed operand: a code can only differ where every input of its 16-token block that is not +0 is -0
    gc, wc = O.unpack_codes(u8(qc.d)), O.unpack_codes(c[0])
    diff = gc != wc
    assert np.all((gc[diff] & 7) == 0) and np.all((wc[diff] & 7) == 0)
    blk_has_negz = negz.T.reshape(C, M // 16, 16).any(-1).repeat(16, axis=1)
    assert np.all(blk_has_negz[diff])
    assert np.array_equal(nvq.dequant(qr).cpu().numpy(), O.dequant(r[0], r[1], r[2]))


def test_tile_quantizer_hadamard_in_the_mma(mods):
    """nvfp4_quant_tile_set_path(2): the 16-point Hadamard transform of the transposed operand is computed by the
    tensor core (B operand = rows of H diag(signs)) instead of FP32 butterflies (the reference's fused backward does
    the same on mma.sync, small-model/fused_bwd.cu:33-64).  The summation order inside the tensor core is its own, so:
    integer-valued inputs (every order exact) must give the oracle's bytes; on Student-t gradients, whose blocks can
    span more than 2^12, codes and scale bytes may differ where the last bit of a sum differs -- stated bound 1e-4 of
    them, by one step; the row operand does not pass through the transform and stays bit-exact."""
    nvq, _, L = mods
    lib = L.load()
    signs = 0xA6B1
    assert lib.nvfp4_quant_tile_set_path(2) == 0
    try:
        rng = np.random.default_rng(5)
        xi = bf16_round(rng.integers(-64, 65, (256, 256)).astype(np.float32))
        r, c = O.quant_rows(xi), O.quant_cols_rht(xi, signs)
        qr, qc = nvq.quant_rows_cols_rht(to_dev(xi), signs)
        check_nvq(qr, r[0], r[1], r[2], 256, 256)
        check_nvq(qc, c[0], c[1], c[2], 256, 256)
        for x in (make_dy(9, 2048, 256), make_x(10, 2048, 384)):
            M, C = x.shape
            r, c = O.quant_rows(x), O.quant_cols_rht(x, signs)
            qr, qc = nvq.quant_rows_cols_rht(to_dev(x), signs)
            check_nvq(qr, r[0], r[1], r[2], M, C)
            got_c, got_s = O.unpack_codes(u8(qc.d)), O.unswizzle_scales(u8(qc.s), C, M // 16)
            want_c = O.unpack_codes(c[0])
            dc, ds = got_c != want_c, got_s != c[1]
            assert dc.mean() <= 1e-4 and ds.mean() <= 1e-4, (dc.mean(), ds.mean())
            assert np.abs((got_c & 7).astype(int) - (want_c & 7).astype(int))[dc].max(initial=0) <= 1
            assert np.abs(got_s.astype(int) - c[1].astype(int)).max() <= 1
            assert qc.gs.item() == float(c[2])
    finally:
        lib.nvfp4_quant_tile_set_path(0)
    assert nvq.quant_tile_status() == 0


def test_tile_quantizer_single_outputs_strided_input_and_device_seeds(mods, tile_path):
    nvq, _, L = mods
    signs = 0x0F0F
    x = make_x(21, 256, 256)
    big = to_dev(np.concatenate([x, x], axis=1))
    view = big[:, 256:]                                   # row stride 512
    r = O.quant_rows(x)
    c = O.quant_cols_rht(x, signs)
    qr, none = nvq.quant_rows_cols_rht(view, signs, want=(True, False))
    assert none is None
    check_nvq(qr, r[0], r[1], r[2], 256, 256)
    none, qc = nvq.quant_rows_cols_rht(view, signs, want=(False, True))
    assert none is None
    check_nvq(qc, c[0], c[1], c[2], 256, 256)
    sd = torch.tensor([77, 78], dtype=torch.int32, device="cuda")
    r = O.quant_rows(x, sr_mode=O.SR_HW, seed=77)
    c = O.quant_cols_rht(x, signs, sr_mode=O.SR_HW, seed=78)
    qr, qc = nvq.quant_rows_cols_rht(view, signs, sr=True, seed=sd[0:1], seed_cols=sd[1:2], sr_mode=L.ROUND_SR_HW)
    check_nvq(qr, r[0], r[1], r[2], 256, 256)
    check_nvq(qc, c[0], c[1], c[2], 256, 256)


def test_fp4ops_fused_operands_equal_the_separate_calls(mods):
    """`fp4ops.quant_rows_cols_rht` (row-major scales, fp4k random stream) against `fp4ops.quant_rows` +
    `fp4ops.quant_cols_rht`, and a weight refreshed in place."""
    _, fp4ops, _ = mods
    g = to_dev(make_dy(31, 256, 192))
    for sr in (False, True):
        a = fp4ops.quant_rows(g, sr=sr, seed=3)
        b = fp4ops.quant_cols_rht(g, 0x1234, sr=sr, seed=4)
        fa, fb = fp4ops.quant_rows_cols_rht(g, 0x1234, sr=sr, seed=3, seed_cols=4)
        assert torch.equal(fa.d, a.d) and torch.equal(fa.s, a.s) and torch.equal(fb.d, b.d) and torch.equal(fb.s, b.s)
        assert fb.k == 4.0 and torch.equal(fa.amax, a.amax)
    w = torch.randn(128, 256, device="cuda")
    q = fp4ops.quant_w2d(w)
    ref = fp4ops.quant_w2d(w * 2)
    same = fp4ops.quant_w2d(w * 2, out=q)
    assert same[0] is q[0] and torch.equal(q[0].d, ref[0].d) and torch.equal(q[1].s, ref[1].s) and torch.equal(q[0].amax, ref[0].amax)


def test_tile_quantizer_rejects_bad_shapes(mods):
    nvq, _, L = mods
    lib = L.load()
    x = torch.zeros(128, 192, dtype=torch.bfloat16, device="cuda")
    am = torch.ones(1, device="cuda")
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    args = lambda M, C: (x.data_ptr(), C, M, C, buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), buf.data_ptr(),
                         L.SCALES_SWIZZLED, am.data_ptr(), None, None, 0, 0, 0, 0, None, None, None)
    assert lib.nvfp4_quant_tile(*args(128, 192)) == -2       # swizzled column scales need C % 128
    assert lib.nvfp4_quant_tile(*args(64, 128)) == -2
    assert lib.nvfp4_quant_tile(*args(0, 128)) == 0


def test_device_side_seed(mods):
    """A seed read from device memory gives the same bits as the same seed passed by value."""
    nvq, _, _ = mods
    x = to_dev(make_dy(6, 128, 128))
    sd = torch.tensor([77], dtype=torch.int32, device="cuda")
    a, b = nvq.quant_rows(x, sr=True, seed=77), nvq.quant_rows(x, sr=True, seed=sd)
    assert torch.equal(a.d.view(torch.uint8), b.d.view(torch.uint8))
    a, b = nvq.quant_cols_rht(x, 3, sr=True, seed=77), nvq.quant_cols_rht(x, 3, sr=True, seed=sd)
    assert torch.equal(a.d.view(torch.uint8), b.d.view(torch.uint8))
    sd.fill_(78)
    c = nvq.quant_cols_rht(x, 3, sr=True, seed=sd)
    assert not torch.equal(a.d.view(torch.uint8), c.d.view(torch.uint8))


def test_swizzle_scales_kernel(mods):
    _, _, L = mods
    rng = np.random.default_rng(0)
    s = rng.integers(0, 256, (256, 40), dtype=np.uint8)
    pad = torch.from_numpy(np.concatenate([s, s], 1)).cuda()
    view = pad[:, 40:]
    out = torch.empty(256 * 40, dtype=torch.uint8, device="cuda")
    L.check(L.load().nvfp4_swizzle_scales(view.data_ptr(), view.stride(0), 256, 40, out.data_ptr(), L.stream()), "swz")
    assert np.array_equal(out.cpu().numpy(), O.swizzle_scales(s))


def test_rejects_bad_arguments(mods):
    nvq, fp4ops, L = mods
    x = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(AssertionError):
        nvq.quant_rows(x[:100])                                  # R % 128 (llm-1b/nvq.py:50)
    with pytest.raises(AssertionError):
        nvq.quant_cols_rht(x, 0)                                 # C % 128 (llm-1b/nvq.py:64)
    with pytest.raises(L.Nvfp4Error):
        nvq.quant_rows(torch.zeros(128, 64, dtype=torch.bfloat16))   # CPU tensor: no fallback
    d = torch.empty(128 * 32 + 1, dtype=torch.uint8, device="cuda")
    s = torch.empty(128 * 4, dtype=torch.uint8, device="cuda")
    am = torch.ones(1, device="cuda")
    lib = L.load()
    assert lib.nvfp4_quant_rows(x.data_ptr(), 64, 128, 64, d.data_ptr() + 1, s.data_ptr(), 0, am.data_ptr(), None, 0, 0, None, L.stream()) == -3
    assert lib.nvfp4_quant_rows(x.data_ptr(), 64, 128, 48, d.data_ptr(), s.data_ptr(), 0, am.data_ptr(), None, 0, 0, None, L.stream()) == -2
    assert lib.nvfp4_quant_rows(x.data_ptr(), 64, 128, 64, d.data_ptr(), s.data_ptr(), 7, am.data_ptr(), None, 0, 0, None, L.stream()) == -4
    assert lib.nvfp4_quant_rows(None, 64, 128, 64, d.data_ptr(), s.data_ptr(), 0, am.data_ptr(), None, 0, 0, None, L.stream()) == -1
