"""GPU parity of the producer-fused emitters (`rms_emit`, `swiglu_emit`) and of `mom_acc` against the oracle's
restatement of llm-1b/emit.cu:97-222, 343-363.

Each producer has one step the CPU cannot model bit for bit, a hardware approximation: rsqrtf in `rms_emit`, __expf and
the approximate division of the sigmoid in `swiglu_emit`.  The kernels hand that intermediate out (rstd per row; the
FP32 activation), so the tests split in two:
  * the approximate step against FP64 within a stated tolerance: rstd within 2^-22 relative (the hardware reciprocal
    square root is specified to about 2^-22.9), the activation within 2e-5 relative + 1e-9 absolute;
  * everything else bit for bit given that intermediate: the residual stream written back, the bf16 outputs, the row
    maxima / per-row scales, scale bytes and codes.
`mom_acc` is integer and IEEE arithmetic only: bit-exact, plus an unbiasedness bound.
"""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from tests.gpu_util import bf16_round, to_dev, u8

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def emit():
    from nvfp4_training_b200 import _lib, emit
    _lib.load()
    yield emit
    _lib.check_status()


def bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def f32_of(t):
    return O.bf16_bits_to_f32(bits(t))


def ulps(a, b):
    """distance in units in the last place between float32 arrays of the same sign"""
    return np.abs(a.view(np.int32).astype(np.int64) - b.view(np.int32).astype(np.int64))


def check_rowq(q, ref, T, C):
    assert np.array_equal(u8(q.d), ref["codes"])
    assert np.array_equal(O.unswizzle_scales(u8(q.s), T, C // 16), ref["scales"])
    assert np.array_equal(q.rs.cpu().numpy().view(np.uint32), ref["rs"].view(np.uint32))


def rms_inputs(seed, T, D):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((T, D)).astype(np.float32) * (1 + 4 * rng.random((T, 1)).astype(np.float32))
    x[:, rng.permutation(D)[:4]] *= 20                         # massive-activation columns
    x = bf16_round(x)
    y = bf16_round(rng.standard_normal((T, D)).astype(np.float32) * 50)       # raw GEMM output, scaled by ys * ygw
    ys = (0.01 + 0.02 * rng.random(T)).astype(np.float32)
    ygw = np.float32(0.731)
    w = bf16_round((1 + 0.2 * rng.standard_normal(D)).astype(np.float32))
    return x, y, ys, ygw, w


@pytest.mark.parametrize("T,D,with_y", [(256, 2048, True), (128, 2048, False), (128, 1024, True), (128, 4096, True)])
def test_rms_emit(emit, T, D, with_y):
    x, y, ys, ygw, w = rms_inputs(T + D, T, D)
    x[7] = 0.0
    if with_y:
        y[7] = 0.0                                             # an all-zero row: rstd = rsqrt(eps), h = 0, codes 0
    q = emit.RowQ(T, D)
    h = torch.empty(T, D, dtype=torch.bfloat16, device="cuda")
    rstd = torch.empty(T, dtype=torch.float32, device="cuda")
    xout = torch.empty(T, D, dtype=torch.bfloat16, device="cuda") if with_y else None
    kw = dict(y=to_dev(y), ys=torch.from_numpy(ys).cuda(), ygw=torch.tensor([ygw], device="cuda"), xout=xout) if with_y else {}
    emit.rms_emit(to_dev(x), to_dev(w), q, h=h, rstd=rstd, eps=1e-5, **kw)
    g_rstd = rstd.cpu().numpy()
    ref = O.rms_emit(x, w, y if with_y else None, ys, ygw, eps=1e-5, rstd=g_rstd)
    # the approximate step: the reciprocal square root against the correctly rounded value
    assert np.abs(g_rstd.astype(np.float64) / ref["rstd_ref"].astype(np.float64) - 1).max() <= 2.0 ** -22
    # everything else bit for bit
    if with_y:
        assert np.array_equal(bits(xout), O.f32_to_bf16_bits(ref["xout"]))
    assert np.array_equal(bits(h), O.f32_to_bf16_bits(ref["h"]))
    check_rowq(q, ref, T, D)
    assert (u8(q.d)[7] == 0).all()
    # the operand alone (no h, no rstd) is the same operand
    q2 = emit.RowQ(T, D)
    emit.rms_emit(to_dev(x), to_dev(w), q2, eps=1e-5, **kw)
    assert torch.equal(q2.d, q.d) and torch.equal(q2.s, q.s) and torch.equal(q2.rs, q.rs)


def test_rms_emit_without_operand_any_row_count(emit):
    """h / rstd only (the reference's bf16 path, llm-1b/model2.py:366-372), T not a multiple of the 8 rows of a CTA."""
    T, D = 100, 2048
    x, y, ys, ygw, w = rms_inputs(5, T, D)
    h = torch.empty(T, D, dtype=torch.bfloat16, device="cuda")
    rstd = torch.empty(T, dtype=torch.float32, device="cuda")
    xout = torch.empty(T, D, dtype=torch.bfloat16, device="cuda")
    emit.rms_emit(to_dev(x), to_dev(w), None, h=h, rstd=rstd, y=to_dev(y), ys=torch.from_numpy(ys).cuda(),
                  ygw=torch.tensor([ygw], device="cuda"), xout=xout)
    ref = O.rms_emit(x, w, y, ys, ygw, rstd=rstd.cpu().numpy())
    assert np.array_equal(bits(xout), O.f32_to_bf16_bits(ref["xout"]))
    assert np.array_equal(bits(h), O.f32_to_bf16_bits(ref["h"]))
    assert np.abs(rstd.cpu().numpy().astype(np.float64) / ref["rstd_ref"].astype(np.float64) - 1).max() <= 2.0 ** -22


def swiglu_inputs(seed, T, F):
    rng = np.random.default_rng(seed)
    gu = bf16_round(rng.standard_normal((T, 2 * F)).astype(np.float32) * 300)      # raw GEMM output
    gu[:, rng.permutation(F)[:3]] *= 8                                              # gates far in the saturated range
    rs_in = (0.002 + 0.004 * rng.random(T)).astype(np.float32)
    return gu, rs_in, np.float32(1.37)


@pytest.mark.parametrize("T,F", [(128, 5632), (256, 2048), (128, 512), (128, 1280)])
def test_swiglu_emit(emit, T, F):
    gu, rs_in, gw = swiglu_inputs(T + F, T, F)
    gu[9] = 0.0
    q = emit.RowQ(T, F)
    a = torch.empty(T, F, dtype=torch.bfloat16, device="cuda")
    a32 = torch.empty(T, F, dtype=torch.float32, device="cuda")
    args = (to_dev(gu), torch.from_numpy(rs_in).cuda(), torch.tensor([gw], device="cuda"))
    emit.swiglu_emit(*args, q, a=a, a_f32=a32)
    g_a = a32.cpu().numpy()
    ref = O.swiglu_emit(gu, rs_in, gw, a_f32=g_a)
    # the approximate step (exponential and division) against FP64
    err = np.abs(g_a.astype(np.float64) - ref["a_ref"].astype(np.float64))
    assert (err <= 2e-5 * np.abs(ref["a_ref"].astype(np.float64)) + 1e-9).all(), float((err / (np.abs(ref["a_ref"]) + 1e-9)).max())
    # everything else bit for bit
    assert np.array_equal(bits(a), O.f32_to_bf16_bits(g_a))
    check_rowq(q, ref, T, F)
    assert (u8(q.d)[9] == 0).all()
    # operand only: same operand
    q2 = emit.RowQ(T, F)
    emit.swiglu_emit(*args, q2)
    assert torch.equal(q2.d, q.d) and torch.equal(q2.s, q.s) and torch.equal(q2.rs, q.rs)
    # tolerance of the whole producer against the FP64 activation: within half a code step of the block plus the
    # approximation error above
    deq = O.emit_rows_dequant(u8(q.d), ref["scales"], ref["rs"])
    step = np.repeat(O.e4m3_decode(ref["scales"]) * ref["rs"][:, None], 16, axis=1)      # value of code 1.0 in each block
    assert (np.abs(deq - ref["a_ref"]) <= 1.0 * step + 1e-6 * np.abs(ref["a_ref"]) + 1e-9).all()


def test_swiglu_emit_activation_only_any_row_count(emit):
    T, F = 130, 5632
    gu, rs_in, gw = swiglu_inputs(3, T, F)
    a = torch.empty(T, F, dtype=torch.bfloat16, device="cuda")
    a32 = torch.empty(T, F, dtype=torch.float32, device="cuda")
    emit.swiglu_emit(to_dev(gu), torch.from_numpy(rs_in).cuda(), torch.tensor([gw], device="cuda"), None, a=a, a_f32=a32)
    assert np.array_equal(bits(a), O.f32_to_bf16_bits(a32.cpu().numpy()))
    ref = O.swiglu_emit(gu, rs_in, gw)
    err = np.abs(a32.cpu().numpy().astype(np.float64) - ref["a_ref"].astype(np.float64))
    assert (err <= 2e-5 * np.abs(ref["a_ref"].astype(np.float64)) + 1e-9).all()


def test_fused_producers_feed_the_gemm(emit):
    """The operands the producers write are what the row-scale GEMM consumes: rms_emit -> gate/up projection ->
    swiglu_emit -> down projection against the FP64 chain on the dequantized operands (llm-1b/model2.py:359-364)."""
    from nvfp4_training_b200 import nvq
    T, D, F = 256, 2048, 512
    x, _, _, _, w = rms_inputs(11, T, D)
    rng = np.random.default_rng(12)
    wgu = bf16_round(rng.standard_normal((2 * F, D)).astype(np.float32) * 0.02)
    wdn = bf16_round(rng.standard_normal((D, F)).astype(np.float32) * 0.02)
    qgu, qdn = emit.WQ(2 * F, D).refresh(to_dev(wgu)), emit.WQ(D, F).refresh(to_dev(wdn))
    hq = emit.rms_emit(to_dev(x), to_dev(w), emit.RowQ(T, D))
    gu_raw = emit.mm_row_w(hq, qgu)                                   # raw: block scales only
    aq = emit.swiglu_emit(gu_raw, hq.rs, qgu.gs, emit.RowQ(T, F))
    out = emit.mm_row_w(aq, qdn, scale=True).float().cpu().numpy()
    # FP64 chain from the same quantized operands
    deq_w = lambda q: nvq.dequant(q).double().cpu().numpy()
    h_deq = emit.dequant(hq.d, hq.s, hq.rs).double().cpu().numpy()
    gu_true = h_deq @ deq_w(qgu.q).T
    g, u = gu_true[:, :F], gu_true[:, F:]
    a_true = g / (1 + np.exp(-g)) * u
    a_deq = emit.dequant(aq.d, aq.s, aq.rs).double().cpu().numpy()
    # the activation operand tracks the FP64 activation within FP4 noise (bf16 raw GEMM output in between)
    assert np.linalg.norm(a_deq - a_true) / np.linalg.norm(a_true) < 0.2
    want = a_deq @ deq_w(qdn.q).T
    assert np.linalg.norm(out - want) / np.linalg.norm(want) <= 4e-3


def test_mom_acc_bit_exact_and_unbiased(emit):
    rng = np.random.default_rng(2)
    n = 8 * 4096 + 8 * 37
    m = bf16_round(rng.standard_normal(n).astype(np.float32) * 0.1)
    g = bf16_round(rng.standard_normal(n).astype(np.float32) * 1e-3)
    m[:8] = 0.0
    alpha, scale, seed, salt = np.float32(0.37), 0.25, 0x1234567, 13
    words = torch.tensor([seed, 0], dtype=torch.int32, device="cuda")
    md = to_dev(m)
    emit.mom_acc(md, to_dev(g), torch.tensor([alpha], device="cuda"), scale, words, salt=salt)
    assert np.array_equal(bits(md), O.f32_to_bf16_bits(O.mom_acc(m, g, alpha, scale, seed, salt)))
    # unbiased: the mean over 256 seeds approaches m + a*g much closer than one bf16 rounding step
    acc = torch.zeros(n, device="cuda")
    gd, al = to_dev(g), torch.tensor([alpha], device="cuda")
    for s in range(256):
        words[0] = s + 1
        md = to_dev(m)
        emit.mom_acc(md, gd, al, scale, words, salt=salt)
        acc += md.float()
    exact = m.astype(np.float64) + float(alpha) * scale * g.astype(np.float64)
    step = np.abs(exact) * 2.0 ** -8 + 1e-30                     # bf16 spacing is at most 2^-7 |x|: half of it
    bias = np.abs((acc / 256).cpu().numpy().astype(np.float64) - exact)
    assert (bias <= 0.45 * step).all()
    assert np.mean(bias / step) < 0.08
