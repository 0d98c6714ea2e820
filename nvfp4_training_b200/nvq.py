"""Drop-in for the reference's `nvq` module (llm-1b/nvq.py): NVFP4 quantizers with swizzled
E4M3 scales and the block-scaled FP4 GEMM, same names, arguments, tensor layouts and assertions,
running on the sm_100a C-ABI library instead of NVRTC kernels + cuBLASLt.

Differences a caller can observe, all inside the stated tolerances:
  * `gs` is `amax / 2688` by IEEE division (the order of small-model/model_ref.py:42), written by the
    quantizer kernel itself, instead of `amax * (1/2688)` (llm-1b/nvq.py:43-44); at most one ulp apart.
  * `mm` applies alpha = gsA*gsB in FP32 inside the GEMM epilogue before the output cast, instead of
    rounding alpha to bf16 and multiplying a bf16 product (llm-1b/nvq.py:96).
  * stochastic rounding defaults to the reference's mantissa-dither method and random stream;
    `SR_MODE` switches to the hardware `cvt.rs` path.
"""
import torch

from . import _lib as L

# rounding used when a quantizer is called with sr=True (a per-call `sr_mode` overrides it):
# ROUND_SR_DITHER = the reference's rounding and random stream, ROUND_SR_HW = hardware cvt.rs
SR_MODE = L.ROUND_SR_DITHER


class Q:
    """Packed NVFP4 matrix [R, C]: d [R, C/2] fp4x2, s swizzled e4m3 (flat), gs = per-tensor scale
    (device, fp32).  Same container as llm-1b/nvq.py:24-29."""
    __slots__ = ("d", "s", "gs")

    def __init__(self, d, s, gs):
        self.d, self.s, self.gs = d, s, gs


def amax(x, out=None, clear=True):
    """max|x| of a contiguous bf16 tensor as a device fp32 [1] (llm-1b/nvq.py:32-40).  `clear=False` (an addition):
    `out` is a word the caller has zeroed, e.g. one of a batch cleared with a single fill, and is only raised."""
    L.require_cuda(x, out)
    if out is None:
        assert clear
        out = torch.empty(1, dtype=torch.float32, device=x.device)
    n = x.numel()
    assert n % 8 == 0 and x.is_contiguous() and x.dtype == torch.bfloat16
    fn = L.load().nvfp4_amax_bf16 if clear else L.load().nvfp4_amax_bf16_update
    L.check(fn(L.ptr(x), n, L.ptr(out), L.stream()), "amax")
    return out


def _new_gs(am):
    # filled by the quantizer kernel with gs = (k*amax)/2688, the role of `_gs` in llm-1b/nvq.py:43-44
    return torch.empty(1, dtype=torch.float32, device=am.device)


def quant_rows(x, sr=False, seed=0, am=None, sr_mode=None):
    """x [R, C] bf16 (row-contiguous) -> Q quantized along C (llm-1b/nvq.py:47-57)."""
    L.require_cuda(x)
    R, C = x.shape
    assert x.dtype == torch.bfloat16
    assert x.stride(1) == 1 and C % 64 == 0 and R % 128 == 0, (R, C)
    if am is None:
        am = amax(x.contiguous())
    d = torch.empty(R, C // 2, dtype=torch.uint8, device=x.device)
    s = torch.empty(R * C // 16, dtype=torch.uint8, device=x.device)
    gs = _new_gs(am)
    L.check(L.load().nvfp4_quant_rows(L.ptr(x), x.stride(0), R, C, L.ptr(d), L.ptr(s), L.SCALES_SWIZZLED, L.ptr(am),
                                      L.ptr(gs), (sr_mode or SR_MODE) if sr else L.ROUND_NEAREST, *L.seed_args(seed), L.stream()),
            "quant_rows")
    return Q(d.view(torch.float4_e2m1fn_x2), s.view(torch.float8_e4m3fn), gs)


def quant_cols_rht(x, signs, sr=False, seed=0, am=None, sr_mode=None):
    """x [M, C] -> Q of x^T [C, M] quantized along M, after a 16-pt RHT along M (llm-1b/nvq.py:60-70)."""
    L.require_cuda(x)
    M, C = x.shape
    assert x.dtype == torch.bfloat16
    x = x.contiguous()
    assert M % 64 == 0 and C % 128 == 0, (M, C)
    if am is None:
        am = amax(x)
    d = torch.empty(C, M // 2, dtype=torch.uint8, device=x.device)
    s = torch.empty(C * M // 16, dtype=torch.uint8, device=x.device)
    gs = _new_gs(am)
    mode = (sr_mode or SR_MODE) if sr else L.ROUND_NEAREST
    if M % 128 == 0:
        # the TMA-staged tile kernel with only the transposed output: same bits, faster than the register-tiled kernel
        host_seed, dev_seed = L.seed_args(seed)
        L.check(L.load().nvfp4_quant_tile(L.ptr(x), C, M, C, None, None, L.ptr(d), L.ptr(s), L.SCALES_SWIZZLED, L.ptr(am),
                                          None, L.ptr(gs), signs & 0xFFFF, mode, 0, host_seed, None, dev_seed, L.stream()),
                "quant_tile")
    else:
        L.check(L.load().nvfp4_quant_cols_rht(L.ptr(x), M, C, L.ptr(d), L.ptr(s), L.SCALES_SWIZZLED, L.ptr(am), L.ptr(gs),
                                              signs & 0xFFFF, mode, *L.seed_args(seed), L.stream()), "quant_cols_rht")
    return Q(d.view(torch.float4_e2m1fn_x2), s.view(torch.float8_e4m3fn), gs)


def quant_rows_cols_rht(x, signs, sr=False, seed=0, seed_cols=0, am=None, sr_mode=None, want=(True, True)):
    """x [M, C] bf16 -> (Q of x along C, Q of x^T along M after the 16-pt RHT): the results of
    `quant_rows(x, ...)` and `quant_cols_rht(x, signs, ...)` (llm-1b/nvq.py:47-70) from one pass
    over x.  `seed` rounds the row operand, `seed_cols` the transposed one; `want` skips an output."""
    L.require_cuda(x)
    M, C = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    assert M % 128 == 0 and C % 128 == 0, (M, C)
    if am is None:
        am = amax(x.contiguous())
    dev = x.device
    qr = qc = None
    dr = sr_ = gr = dc = sc = gc = None
    if want[0]:
        dr = torch.empty(M, C // 2, dtype=torch.uint8, device=dev)
        sr_ = torch.empty(M * C // 16, dtype=torch.uint8, device=dev)
        gr = _new_gs(am)
        qr = Q(dr.view(torch.float4_e2m1fn_x2), sr_.view(torch.float8_e4m3fn), gr)
    if want[1]:
        dc = torch.empty(C, M // 2, dtype=torch.uint8, device=dev)
        sc = torch.empty(C * M // 16, dtype=torch.uint8, device=dev)
        gc = _new_gs(am)
        qc = Q(dc.view(torch.float4_e2m1fn_x2), sc.view(torch.float8_e4m3fn), gc)
    seed_r, seed_r_dev = L.seed_args(seed)
    seed_c, seed_c_dev = L.seed_args(seed_cols)
    L.check(L.load().nvfp4_quant_tile(L.ptr(x), x.stride(0), M, C, L.ptr(dr), L.ptr(sr_), L.ptr(dc), L.ptr(sc),
                                      L.SCALES_SWIZZLED, L.ptr(am), L.ptr(gr), L.ptr(gc), signs & 0xFFFF,
                                      (sr_mode or SR_MODE) if sr else L.ROUND_NEAREST, seed_r, seed_c, seed_r_dev, seed_c_dev,
                                      L.stream()), "quant_tile")
    return qr, qc


def quant_tile_status(reset=True):
    """Status word of the tile quantizer on the current device (0 = no wait ever expired)."""
    import ctypes
    out = ctypes.c_int(0)
    L.check(L.load().nvfp4_quant_tile_status(ctypes.byref(out), 1 if reset else 0), "quant_tile_status")
    return out.value


def quant_w2d(w, am=None, want=(True, True), out=None):
    """w [N, K] bf16 -> (Q of w, Q of w^T), identical values (16x16 blocks) (llm-1b/nvq.py:73-87).
    `want` lets a caller skip one of the two outputs (its slot is then None); `out` = a pair
    returned by an earlier call, overwritten in place (a per-step weight cache keeps its buffers)."""
    L.require_cuda(w)
    N, K = w.shape
    assert w.dtype == torch.bfloat16
    w = w.contiguous()
    assert N % 128 == 0 and K % 128 == 0, (N, K)
    f4, f8 = torch.float4_e2m1fn_x2, torch.float8_e4m3fn
    if out is not None:
        oq, oqt = out
        want = (oq is not None, oqt is not None)
        g = (oq or oqt).gs
        if am is None:
            am = amax(w)
        q, s = (oq.d, oq.s) if oq is not None else (None, None)
        qt, st = (oqt.d, oqt.s) if oqt is not None else (None, None)
    else:
        if am is None:
            am = amax(w)
        g = _new_gs(am)
        q = s = qt = st = None
        if want[0]:
            q = torch.empty(N, K // 2, dtype=torch.uint8, device=w.device).view(f4)
            s = torch.empty(N * K // 16, dtype=torch.uint8, device=w.device).view(f8)
        if want[1]:
            qt = torch.empty(K, N // 2, dtype=torch.uint8, device=w.device).view(f4)
            st = torch.empty(K * N // 16, dtype=torch.uint8, device=w.device).view(f8)
    L.check(L.load().nvfp4_quant_w2d(L.ptr(w), L.DTYPE_BF16, N, K, L.ptr(q), L.ptr(s), L.ptr(qt), L.ptr(st),
                                     L.SCALES_SWIZZLED, L.ptr(am), L.ptr(g), L.stream()), "quant_w2d")
    if out is not None:
        return out
    return (Q(q, s, g) if want[0] else None, Q(qt, st, g) if want[1] else None)


def mm(a: Q, b: Q, out_dtype=torch.bfloat16, scale=True, out=None, accumulate=False, splitk=1, owners=None):
    """a [M,K], b [N,K] (both K-major) -> a @ b^T [M, N].  If scale=False returns (raw, alpha)
    (llm-1b/nvq.py:90-96).  `out` / `accumulate` (fp32 only) are additions for in-place wgrad; `splitk=0` (fp32 only)
    lets the library slice a long contraction over the SMs (sums then land in no fixed order).
    `owners` (fp32 `out` only): the addresses of `out` on every data-parallel rank (peer mappings; this rank's own
    `out.data_ptr()` at its index); the product is then added into the row slab each rank owns instead of into `out`
    (`nvfp4_gemm_scatter_rows`)."""
    M, N, K = a.d.shape[0], b.d.shape[0], a.d.shape[1] * 2
    assert b.d.shape[1] * 2 == K, (a.d.shape, b.d.shape)
    assert out_dtype in (torch.bfloat16, torch.float32)
    L.require_cuda(a.d, b.d)
    if out is None:
        assert not accumulate and owners is None
        out = torch.empty(M, N, dtype=out_dtype, device=a.d.device)
    else:
        assert out.shape == (M, N) and out.dtype == out_dtype and out.stride(1) == 1
    if owners is not None:
        assert out_dtype == torch.float32
        L.check(L.load().nvfp4_gemm_scatter_rows(L.ptr(a.d), L.ptr(a.s), a.d.stride(0), L.ptr(b.d), L.ptr(b.s), b.d.stride(0),
                                                 L.ptr_array(owners), len(owners), out.stride(0), M, N, K,
                                                 L.ALPHA_GS if scale else L.ALPHA_ONE, L.ptr(a.gs) if scale else None,
                                                 L.ptr(b.gs) if scale else None, 1.0, 1.0, splitk,
                                                 L.ptr(L.status_word(a.d.device)), L.stream()), "mm (scatter)")
        return out
    L.check(L.load().nvfp4_gemm(L.ptr(a.d), L.ptr(a.s), a.d.stride(0), L.ptr(b.d), L.ptr(b.s), b.d.stride(0),
                                L.ptr(out), L.DTYPE_FP32 if out_dtype == torch.float32 else L.DTYPE_BF16,
                                out.stride(0), M, N, K, L.ALPHA_GS if scale else L.ALPHA_ONE,
                                L.ptr(a.gs) if scale else None, L.ptr(b.gs) if scale else None, 1.0, 1.0,
                                int(accumulate), splitk if out_dtype == torch.float32 else 1,
                                L.ptr(L.status_word(a.d.device)), L.stream()), "mm")
    if not scale:
        return out, a.gs * b.gs
    return out


# ---------- reference decode (tests), llm-1b/nvq.py:99-117
_E2M1 = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6])


def unswizzle(s, R, C16):
    ncb = C16 // 4
    t = s.view(torch.uint8).reshape(R // 128, ncb, 32, 4, 4)       # rb, cb, r%32, (r%128)/32, c%4
    return t.permute(0, 3, 2, 1, 4).reshape(R, C16)                 # rb,(r/32),(r%32), cb, c%4


def dequant(q: Q):
    d = q.d.view(torch.uint8)
    R, C = d.shape[0], d.shape[1] * 2
    lo, hi = (d & 15).long(), (d >> 4).long()
    tab = _E2M1.to(d.device)
    v = torch.stack([tab[lo], tab[hi]], -1).reshape(R, C)
    s = unswizzle(q.s, R, C // 16).view(torch.float8_e4m3fn).float().repeat_interleave(16, 1)
    return v * s * q.gs
