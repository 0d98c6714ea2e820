"""Drop-in for the reference's `fp4ops` module (llm-1b/fp4ops.py = small-model/fp4ops.py):
quantizers with row-major `[R, C/16]` scales, FP32 weights, and `gemm` with bf16 output or FP32
split-K accumulation, on the sm_100a C-ABI library.

The tensor-core path consumes swizzled scales, so `gemm` first rewrites the operands' scales into
a scratch buffer it allocates with torch (the C entry point takes it as `workspace`).  An operand whose
swizzled scales are already known (`Q.sw`, kept by `fp4torch.FP4Weight` for the weights) skips that step.
"""
import weakref

import torch

from . import _lib as L

SMEM_GEMM = 6 * (128 * 128 + 128 * 128 + 2048 + 2048) + 1280   # informational, like llm-1b/fp4ops.py:8
SR_MODE = L.ROUND_SR_DITHER_K


class Q:
    """Packed NVFP4 tensor: data [R, C/2] uint8, scales [R, C/16] uint8, amax (device scalar),
    k (extra scale) (llm-1b/fp4ops.py:18-23)."""
    __slots__ = ("d", "s", "amax", "k", "sw")

    def __init__(self, d, s, amax, k=1.0, sw=None):
        self.d, self.s, self.amax, self.k = d, s, amax, k
        self.sw = sw        # optional: the same scales in the 128x4-tile swizzled layout (an addition of this library)


def swizzle_scales(s, out=None):
    """Row-major scales [R, C/16] (row stride honoured) -> the swizzled layout the tensor core reads, flat uint8."""
    R, C16 = s.shape
    assert R % 128 == 0 and C16 % 4 == 0, (R, C16)
    if out is None:
        out = torch.empty(R * C16, dtype=torch.uint8, device=s.device)
    L.check(L.load().nvfp4_swizzle_scales(L.ptr(s), s.stride(0), R, C16, L.ptr(out), L.stream()), "swizzle_scales")
    return out


# Swizzled scale copies of long-lived operands (weights), found by the address of their row-major scales: the
# torch custom ops of fp4torch receive plain tensors, not Q objects.  An entry is valid while the tensor it was
# made from is alive (its memory cannot have been reused) and is rewritten by whoever rewrites that tensor.
_SW_CACHE = {}


def remember_swizzled(s, sw):
    _SW_CACHE[s.data_ptr()] = (weakref.ref(s), sw)
    if len(_SW_CACHE) > 4096:
        for k in [k for k, (r, _) in _SW_CACHE.items() if r() is None]:
            del _SW_CACHE[k]


def swizzled_of(s):
    e = _SW_CACHE.get(s.data_ptr())
    if e is None:
        return None
    t = e[0]()
    if t is None or t.data_ptr() != s.data_ptr() or t.shape != s.shape or t.stride() != s.stride():
        return None
    return e[1]


def amax_of(x):
    """max|x| as a device fp32 [1] (llm-1b/fp4ops.py:25-26).  bf16 inputs take the one-read amax kernel
    (same value); other dtypes, e.g. FP32 master weights once per step, the torch reduction."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.numel() % 8 == 0 and x.numel() > 0:
        out = torch.empty(1, dtype=torch.float32, device=x.device)
        L.check(L.load().nvfp4_amax_bf16(L.ptr(x), x.numel(), L.ptr(out), L.stream()), "amax")
        return out
    return x.abs().amax().float().reshape(1)


def quant_rows(x, sr=False, seed=0, amax=None):
    """llm-1b/fp4ops.py:30-38."""
    L.require_cuda(x)
    R, C = x.shape
    x = x.contiguous()
    assert x.dtype == torch.bfloat16 and C % 16 == 0
    a = amax_of(x) if amax is None else amax
    d = torch.empty(R, C // 2, dtype=torch.uint8, device=x.device)
    s = torch.empty(R, C // 16, dtype=torch.uint8, device=x.device)
    L.check(L.load().nvfp4_quant_rows(L.ptr(x), C, R, C, L.ptr(d), L.ptr(s), L.SCALES_LINEAR, L.ptr(a),
                                      None, SR_MODE if sr else L.ROUND_NEAREST, *L.seed_args(seed), L.stream()), "quant_rows")
    return Q(d, s, a)


def quant_cols_rht(x, signs, sr=False, seed=0, amax=None):
    """x [M, C] -> quantized along M of x^T: data [C, M/2].  RHT applied along M (16-blocks)
    (llm-1b/fp4ops.py:41-49)."""
    L.require_cuda(x)
    M, C = x.shape
    x = x.contiguous()
    assert x.dtype == torch.bfloat16 and M % 16 == 0 and C % 8 == 0
    a = amax_of(x) if amax is None else amax
    d = torch.empty(C, M // 2, dtype=torch.uint8, device=x.device)
    s = torch.empty(C, M // 16, dtype=torch.uint8, device=x.device)
    L.check(L.load().nvfp4_quant_cols_rht(L.ptr(x), M, C, L.ptr(d), L.ptr(s), L.SCALES_LINEAR, L.ptr(a), None, signs & 0xFFFF,
                                          SR_MODE if sr else L.ROUND_NEAREST, *L.seed_args(seed), L.stream()),
            "quant_cols_rht")
    return Q(d, s, a, 4.0)


def quant_rows_cols_rht(x, signs, sr=False, seed=0, seed_cols=0, amax=None):
    """Both operands of one activation / gradient from a single pass over it: what
    `quant_rows(x, sr, seed, amax)` and `quant_cols_rht(x, signs, sr, seed_cols, amax)` return
    (llm-1b/fp4ops.py:30-49), bit for bit.  Needs M % 128 == 0 and C % 64 == 0."""
    L.require_cuda(x)
    M, C = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and M % 128 == 0 and C % 64 == 0, (M, C)
    a = amax_of(x) if amax is None else amax
    dev = x.device
    dr = torch.empty(M, C // 2, dtype=torch.uint8, device=dev)
    sr_ = torch.empty(M, C // 16, dtype=torch.uint8, device=dev)
    dc = torch.empty(C, M // 2, dtype=torch.uint8, device=dev)
    sc = torch.empty(C, M // 16, dtype=torch.uint8, device=dev)
    s_r, s_r_dev = L.seed_args(seed)
    s_c, s_c_dev = L.seed_args(seed_cols)
    L.check(L.load().nvfp4_quant_tile(L.ptr(x), x.stride(0), M, C, L.ptr(dr), L.ptr(sr_), L.ptr(dc), L.ptr(sc), L.SCALES_LINEAR,
                                      L.ptr(a), None, None, signs & 0xFFFF, SR_MODE if sr else L.ROUND_NEAREST, s_r, s_c,
                                      s_r_dev, s_c_dev, L.stream()), "quant_tile")
    return Q(dr, sr_, a), Q(dc, sc, a, 4.0)


def quant_w2d(w, out=None):
    """w fp32 [N, K] -> (Q, Q^T) (llm-1b/fp4ops.py:52-61).  `out`: a pair returned earlier, rewritten in
    place (its amax included), so that holders of the buffers see the refreshed weight."""
    L.require_cuda(w)
    N, K = w.shape
    assert w.dtype == torch.float32 and N % 16 == 0 and K % 16 == 0
    if out is None:
        mk = lambda r, c: torch.empty(r, c, dtype=torch.uint8, device=w.device)
        a = torch.empty(1, dtype=torch.float32, device=w.device)
        out = (Q(mk(N, K // 2), mk(N, K // 16), a), Q(mk(K, N // 2), mk(K, N // 16), a))
    qw, qwt = out
    qw.amax.copy_(amax_of(w))
    L.check(L.load().nvfp4_quant_w2d(L.ptr(w.contiguous()), L.DTYPE_FP32, N, K, L.ptr(qw.d), L.ptr(qw.s), L.ptr(qwt.d),
                                     L.ptr(qwt.s), L.SCALES_LINEAR, L.ptr(qw.amax), None, L.stream()), "quant_w2d")
    for q in (qw, qwt):
        if q.sw is not None:        # a rewritten pair keeps its swizzled scale copies in step
            swizzle_scales(q.s, out=q.sw)
    return qw, qwt


def gemm(a: Q, b: Q, out=None, splitk=1):
    """a: [M,K] fp4, b: [N,K] fp4 -> [M,N].  splitk>1 or out given -> fp32 atomic accumulate into out
    (llm-1b/fp4ops.py:64-80).  Row strides of d and s are honoured."""
    L.require_cuda(a.d, b.d)
    M, N, K = a.d.shape[0], b.d.shape[0], a.s.shape[1] * 16
    assert M % 128 == 0 and N % 128 == 0 and K % 128 == 0, (M, N, K)
    if splitk == 1 and out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.d.device)
        acc, cdt = 0, L.DTYPE_BF16
    else:
        if out is None:
            out = torch.zeros(M, N, dtype=torch.float32, device=a.d.device)
        assert out.dtype == torch.float32 and out.stride(1) == 1
        acc, cdt = 1, L.DTYPE_FP32
    lib = L.load()
    sw_a = a.sw if a.sw is not None else swizzled_of(a.s)
    sw_b = b.sw if b.sw is not None else swizzled_of(b.s)
    if sw_a is None and sw_b is None:
        ws = torch.empty(lib.nvfp4_gemm_linear_workspace_bytes(M, N, K), dtype=torch.uint8, device=a.d.device)
        L.check(lib.nvfp4_gemm_linear(L.ptr(a.d), L.ptr(a.s), a.d.stride(0), a.s.stride(0), L.ptr(b.d), L.ptr(b.s),
                                      b.d.stride(0), b.s.stride(0), L.ptr(out), cdt, out.stride(0), M, N, K, L.ALPHA_AMAX,
                                      L.ptr(a.amax), L.ptr(b.amax), float(a.k), float(b.k), acc, splitk, L.ptr(ws),
                                      ws.numel(), L.ptr(L.status_word(a.d.device)), L.stream()), "gemm")
        return out
    # at least one operand brings its swizzled scales: swizzle the other and call the swizzled-scale GEMM
    if sw_a is None:
        sw_a = swizzle_scales(a.s)
    if sw_b is None:
        sw_b = swizzle_scales(b.s)
    L.check(lib.nvfp4_gemm(L.ptr(a.d), L.ptr(sw_a), a.d.stride(0), L.ptr(b.d), L.ptr(sw_b), b.d.stride(0), L.ptr(out), cdt,
                           out.stride(0), M, N, K, L.ALPHA_AMAX, L.ptr(a.amax), L.ptr(b.amax), float(a.k), float(b.k), acc,
                           splitk, L.ptr(L.status_word(a.d.device)), L.stream()), "gemm")
    return out


# ---------- reference decode (for tests), llm-1b/fp4ops.py:83-92
_E2M1 = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6])


def dequant(q: Q):
    d = q.d
    lo, hi = (d & 15).long(), (d >> 4).long()
    v = torch.stack([_E2M1.to(d.device)[lo], _E2M1.to(d.device)[hi]], -1).reshape(d.shape[0], -1)
    s = q.s.view(torch.float8_e4m3fn).float().repeat_interleave(16, 1)
    return v * s * (q.amax * q.k / 2688.0)
