"""Operand emitters of the reference's 1B trainer (llm-1b/emit.py) on the sm_100a library: the
row operand with an exact per-row FP32 scale, so no tensor-wide amax pass precedes it, and the raw
block-scaled GEMM whose result the consumer multiplies by `rs[t] * gs`.

Built: `RowQ`, `ColQ`, `row_emit`, `col_emit`, `rms_emit`, `swiglu_emit`, `mom_acc`, `WQ`, `mm`, `mm_row_w`, `mm_row_wt`,
`mm_col`, `scale_rows`, `dequant`.
`mm_row_w` / `mm_row_wt` / `mm_col` take `scale=True` to apply `rs[row] * gs` (resp. the two delayed tensor scales) in
the GEMM epilogue, which the reference does in a separate elementwise pass (`scale_rows`, llm-1b/model2.py:152-154).
"""
import torch

from . import _lib as L
from . import nvq

F4, F8 = torch.float4_e2m1fn_x2, torch.float8_e4m3fn


class RowQ:
    """Row operand [R, C]: data (fp4x2 [R, C/2]), swizzled scales, rs[R] per-row fp32 scale
    (llm-1b/emit.py:20-27)."""
    __slots__ = ("d", "s", "rs")

    def __init__(self, R, C, dev="cuda"):
        self.d = torch.empty(R, C // 2, dtype=torch.uint8, device=dev)
        self.s = torch.empty(R * C // 16, dtype=torch.uint8, device=dev)
        self.rs = torch.empty(R, dtype=torch.float32, device=dev)


class ColQ:
    """Column operand of X [M, C]: X^T quantized along M -> data [C, M/2], swizzled scales
    (llm-1b/emit.py:30-36)."""
    __slots__ = ("d", "s")

    def __init__(self, M, C, dev="cuda"):
        self.d = torch.empty(C, M // 2, dtype=torch.uint8, device=dev)
        self.s = torch.empty(C * M // 16, dtype=torch.uint8, device=dev)


def col_emit(x, q: ColQ, amax_use, amax_cur, rng, sr=False, salt=0):
    """RHT16 along the tokens + quantization of x^T with the delayed scale `amax_use`; records the
    RHT-domain amax of x into `amax_cur` (float bits, atomicMax: zero it first) (llm-1b/emit.py:82-85).
    `rng`: CUDA int32 words, rng[0] = SR seed, rng[1] = Hadamard sign bits.  `sr`: False / True (the reference's
    dither and sequence) / "hw" (hardware stochastic convert, this library's counter-based words)."""
    L.require_cuda(x, q.d, q.s, amax_use, amax_cur, rng)
    M, C = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and M % 256 == 0 and C % 64 == 0
    assert C % 128 == 0, C          # swizzled scale tiles of 128 columns are written whole
    assert rng.element_size() == 4 and rng.numel() >= 2 and amax_cur.element_size() == 4
    L.check(L.load().nvfp4_emit_cols(L.ptr(x), x.stride(0), M, C, L.ptr(q.d), L.ptr(q.s), L.ptr(amax_use), L.ptr(amax_cur),
                                     2 if sr == "hw" else int(bool(sr)), L.ptr(rng), salt & 0xFFFFFFFF, L.stream()), "emit_cols")
    return q


def row_emit(x, q: RowQ, rng, sr=False, salt=0):
    """Quantize the rows of x [T, C] into q (llm-1b/emit.py:72-79).  `rng`: CUDA int32/uint32 words,
    rng[0] = stochastic-rounding seed (read on the device, so a captured graph sees fresh seeds).
    `sr`: False = round to nearest, True = the reference's mantissa dither and random sequence, "hw" = the hardware
    stochastic convert with this library's counter-based words (an addition)."""
    L.require_cuda(x, q.d, q.s, q.rs)
    T, C = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and C % 256 == 0
    assert T % 128 == 0, T
    if sr:
        assert rng is not None and rng.is_cuda and rng.element_size() == 4
    L.check(L.load().nvfp4_emit_rows(L.ptr(x), x.stride(0), T, C, L.ptr(q.d), L.ptr(q.s), L.ptr(q.rs), 2 if sr == "hw" else int(bool(sr)),
                                     L.ptr(rng) if rng is not None else None, salt & 0xFFFFFFFF, L.stream()), "emit_rows")
    return q


def rms_emit(x, w, q: RowQ = None, h=None, rstd=None, y=None, ys=None, ygw=None, xout=None, eps=1e-5):
    """Residual add + RMSNorm + row quantization in one pass (llm-1b/emit.py:40-47, llm-1b/emit.cu:97-147):
    x_new = x + y * ys[t] * ygw (written to `xout`), hn = x_new * rstd * w -> row operand `q`; optional `h` (bf16 hn)
    and `rstd` (fp32 [T]) outputs.  x [T, D] contiguous bf16 with D in {1024, 2048, 4096} (the reference: 2048)."""
    T, D = x.shape
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and w.dtype == torch.bfloat16 and w.numel() == D
    L.require_cuda(x, w)
    if y is not None:
        assert y.shape == x.shape and y.is_contiguous() and ys is not None and ygw is not None and xout is not None
        assert xout.shape == x.shape and xout.is_contiguous() and ys.dtype == torch.float32 and ygw.dtype == torch.float32
    if q is not None:
        assert T % 128 == 0 and q.d.shape == (T, D // 2)
    if h is not None:
        assert h.shape == x.shape and h.is_contiguous() and h.dtype == torch.bfloat16
    o = lambda t: L.ptr(t) if t is not None else None
    L.check(L.load().nvfp4_rms_emit(L.ptr(x), o(y), o(ys), o(ygw), o(xout), L.ptr(w), o(h), o(q.d if q else None),
                                    o(q.s if q else None), o(q.rs if q else None), o(rstd), T, D, float(eps), L.stream()),
            "rms_emit")
    return q


def swiglu_emit(gu, rs_in, gw, q: RowQ = None, a=None, a_f32=None):
    """SwiGLU on the raw gate | up GEMM output [T, 2F] + row quantization of a = silu(g) * u, true g, u = raw *
    rs_in[t] * gw (llm-1b/emit.py:50-58, llm-1b/emit.cu:149-222).  Optional `a` (bf16 [T, F]); `a_f32` (fp32 [T, F],
    an addition for tests: the values that are quantized)."""
    T, F2 = gu.shape
    F = F2 // 2
    assert gu.dtype == torch.bfloat16 and gu.is_contiguous() and F2 % 512 == 0
    assert rs_in.dtype == torch.float32 and rs_in.numel() == T and gw.dtype == torch.float32
    L.require_cuda(gu, rs_in, gw)
    if q is not None:
        assert T % 128 == 0 and q.d.shape == (T, F // 2)
    o = lambda t: L.ptr(t) if t is not None else None
    L.check(L.load().nvfp4_swiglu_emit(L.ptr(gu), L.ptr(rs_in), L.ptr(gw), F, o(a), o(a_f32), o(q.d if q else None),
                                       o(q.s if q else None), o(q.rs if q else None), T, L.stream()), "swiglu_emit")
    return q


def mom_acc(m, g, alpha, scale, rng, salt=0):
    """m (bf16) += alpha * scale * g (bf16), stochastically rounded (llm-1b/emit.py:77-80, llm-1b/emit.cu:343-363).
    alpha: device fp32 [1]; rng: device int32 words, rng[0] = seed."""
    n = m.numel()
    assert n % 8 == 0 and g.numel() == n and m.dtype == torch.bfloat16 and g.dtype == torch.bfloat16
    assert m.is_contiguous() and g.is_contiguous() and alpha.dtype == torch.float32
    L.require_cuda(m, g, alpha, rng)
    L.check(L.load().nvfp4_mom_acc(L.ptr(m), L.ptr(g), L.ptr(alpha), float(scale), n, L.ptr(rng), salt & 0xFFFFFFFF, L.stream()),
            "mom_acc")
    return m


class WQ:
    """FP4 form of a weight W [N, K] and of W^T, per-tensor scale gs = amax/2688 (llm-1b/emit.py:100-128).
    The reference re-quantizes just in time into a scratch shared by same-shape weights; here
    `refresh` quantizes once per optimizer step into buffers the object owns."""

    def __init__(self, N, K, dev="cuda"):
        self.N, self.K = N, K
        self.q = self.qt = None

    def refresh(self, w):
        w = w.detach().to(torch.bfloat16)
        if self.q is None:
            self.q, self.qt = nvq.quant_w2d(w)
        else:
            nvq.quant_w2d(w, out=(self.q, self.qt))
        return self

    def prep(self):
        return self

    @property
    def gs(self):
        return self.q.gs

    d = property(lambda self: self.q.d)
    s = property(lambda self: self.q.s)
    td = property(lambda self: self.qt.d)
    ts = property(lambda self: self.qt.s)


_ONES = {}


def _one(dev):
    if dev not in _ONES:
        _ONES[dev] = torch.ones(1, dtype=torch.float32, device=dev)
    return _ONES[dev]


def mm(ad, as_, bd, bs, out_dtype=torch.bfloat16):
    """raw = A @ B^T with block scales only; A [M, K], B [N, K] fp4 row-major (llm-1b/emit.py:131-133)."""
    one = _one(ad.device)
    a = nvq.Q(ad.view(F4), as_.view(F8), one)
    b = nvq.Q(bd.view(F4), bs.view(F8), one)
    return nvq.mm(a, b, out_dtype=out_dtype, scale=False)[0]


def _gemm(ad, as_, bd, bs, out, alpha_mode, pa, pb, accumulate=False, splitk=1, owners=None):
    M, N, K = ad.shape[0], bd.shape[0], ad.shape[1] * 2
    assert bd.shape[1] * 2 == K and out.shape == (M, N) and out.stride(1) == 1
    L.require_cuda(ad, bd, out)
    if owners is not None:       # add into the row slab every rank owns (nvq.mm's `owners`)
        assert out.dtype == torch.float32
        L.check(L.load().nvfp4_gemm_scatter_rows(L.ptr(ad), L.ptr(as_), ad.stride(0), L.ptr(bd), L.ptr(bs), bd.stride(0),
                                                 L.ptr_array(owners), len(owners), out.stride(0), M, N, K, alpha_mode,
                                                 L.ptr(pa), L.ptr(pb), 1.0, 1.0, splitk,
                                                 L.ptr(L.status_word(ad.device)), L.stream()), "gemm (scatter)")
        return out
    L.check(L.load().nvfp4_gemm(L.ptr(ad), L.ptr(as_), ad.stride(0), L.ptr(bd), L.ptr(bs), bd.stride(0), L.ptr(out),
                                L.DTYPE_FP32 if out.dtype == torch.float32 else L.DTYPE_BF16, out.stride(0), M, N, K,
                                alpha_mode, L.ptr(pa), L.ptr(pb), 1.0, 1.0, int(accumulate), splitk,
                                L.ptr(L.status_word(ad.device)), L.stream()), "gemm")
    return out


def scale_rows(raw, rs, gs):
    """true = raw * rs[:, None] * gs as bf16: the reference's separate pass (llm-1b/model2.py:152-154)."""
    return (raw.float() * (rs[:, None] * gs)).to(torch.bfloat16)


def dequant(d, s, rs):
    """Row operand back to FP32 [R, C] (tests; `E.dequant` of llm-1b/test_emit.py)."""
    R, C = d.shape[0], d.shape[1] * 2
    return nvq.dequant(nvq.Q(d.view(F4), s.view(F8), _one(d.device))) * rs[:, None]


def mm_col(a: ColQ, b: ColQ, out_dtype=torch.float32, scale=False, amax_a=None, amax_b=None, out=None, accumulate=False,
           owners=None):
    """wgrad: dW_raw = Q(H dy)^T Q(H x) [N, K]; true = raw * gsA * gsB with gs = amax_use/2688
    (llm-1b/emit.py:148-150).  scale=True: the two delayed amax words (device fp32 [1]) are given and
    the product by gsA * gsB happens in the epilogue; `out` / `accumulate`: in-place FP32 accumulation."""
    if not scale:
        return mm(a.d, a.s, b.d, b.s, out_dtype=out_dtype)
    if out is None:
        out = torch.empty(a.d.shape[0], b.d.shape[0], dtype=out_dtype, device=a.d.device)
    return _gemm(a.d, a.s, b.d, b.s, out, L.ALPHA_AMAX, amax_a, amax_b, accumulate,
                 splitk=0 if out.dtype == torch.float32 else 1, owners=owners)


def mm_row_w(q: RowQ, w: WQ, scale=False):
    """forward: y_raw = Q(x) @ Q(W)^T; true y = y_raw * q.rs[:, None] * w.gs (llm-1b/emit.py:136-140).
    scale=True returns the true y (bf16), scaled per row in the GEMM epilogue."""
    if not scale:
        return mm(q.d, q.s, w.d, w.s)
    out = torch.empty(q.d.shape[0], w.d.shape[0], dtype=torch.bfloat16, device=q.d.device)
    return _gemm(q.d, q.s, w.d, w.s, out, L.ALPHA_ROW, q.rs, w.gs)


def mm_row_wt(q: RowQ, w: WQ, scale=False):
    """dgrad: dx_raw = Q(dy) @ Q(W); true = raw * q.rs[:, None] * w.gs (llm-1b/emit.py:143-145)."""
    if not scale:
        return mm(q.d, q.s, w.td, w.ts)
    out = torch.empty(q.d.shape[0], w.td.shape[0], dtype=torch.bfloat16, device=q.d.device)
    return _gemm(q.d, q.s, w.td, w.ts, out, L.ALPHA_ROW, q.rs, w.gs)
