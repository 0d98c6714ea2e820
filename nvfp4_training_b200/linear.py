"""Autograd NVFP4 linear layer: the recipe of `FP4LinearFn` / `Linear` in the reference
(llm-1b/model.py:36-90) on the sm_100a kernels.

  fprop : y  = Q_rn(x)  @ Q2d(W)^T
  dgrad : dx = Q_sr(dy) @ Q2d(W)          (W^T operand: same 16x16-block values)
  wgrad : dW = Q_sr(H dy)^T @ Q_rn(H x)   (16-point random Hadamard along tokens)

Additions that do not change results: `LinCtx.wgrad_dtype` (the reference returns a bf16 weight
gradient, llm-1b/nvq.py:90; FP32 is what a data-parallel all-reduce wants) and `WeightCache`, which
quantizes a weight once per optimizer step instead of twice per microbatch -- the scheme of
`FP4Weight.refresh` (small-model/fp4torch.py:71-84).
"""
import torch
import torch.nn as nn

from . import nvq


class LinCtx:
    """Global switches for the linear layers (llm-1b/model.py:36-39)."""
    fp4 = True
    seed = 0                       # changes every microbatch (stochastic rounding)
    wgrad_dtype = torch.bfloat16   # reference default; torch.float32 for FP32 weight gradients


_RHT_SIGNS = 0b1010011010110001    # llm-1b/model.py:42


def sr_seed(lid):
    """Per-layer, per-microbatch seed (llm-1b/model.py:59)."""
    return (LinCtx.seed * 1000003 + lid * 7919) & 0xFFFFFFFF


class WeightCache:
    """Quantized W and W^T of one weight, refreshed once per optimizer step."""

    def __init__(self, weight):
        self.weight = weight
        self.q = self.qt = None

    @torch.no_grad()
    def refresh(self):
        self.q, self.qt = nvq.quant_w2d(self.weight.detach().to(torch.bfloat16))
        return self


def _tileable(t):
    """Shapes the one-read tile quantizer takes (else the row and column kernels run separately)."""
    return t.shape[0] % 128 == 0 and t.shape[1] % 128 == 0


def linear_fwd(x, qw, keep_xt=False, signs=_RHT_SIGNS, am_out=None):
    """fprop of llm-1b/model.py:46-53 with W already quantized: returns (y bf16 [T, N], amax(x)).
    amax(x) is handed back so the backward pass does not recompute it (same value).  With
    `keep_xt` the transposed RHT operand of x that wgrad needs (llm-1b/model.py:66) is produced in
    the same pass over x and returned as a third value, so the backward pass neither re-reads nor
    has to keep x.  `am_out`: a zeroed device word that receives amax(x) (callers that clear many such words with
    one fill save a fill per call)."""
    am = nvq.amax(x.contiguous()) if am_out is None else nvq.amax(x.contiguous(), out=am_out, clear=False)
    if keep_xt and _tileable(x):
        qx, qxt = nvq.quant_rows_cols_rht(x, signs, am=am)
        return nvq.mm(qx, qw), am, qxt
    y = nvq.mm(nvq.quant_rows(x, am=am), qw)
    return (y, am, nvq.quant_cols_rht(x, signs, am=am)) if keep_xt else (y, am)


def linear_bwd(x, am_x, gy, qwt, seed, seed_cols, gw_out=None, wgrad_dtype=torch.float32, signs=_RHT_SIGNS,
               sr_mode=None, overwrite=False, qxt=None, am_gy=None, wgrad_stream=None, keep_alive=None, am_out=None,
               gw_owners=None):
    """dgrad + wgrad of llm-1b/model.py:55-69.  `seed` / `seed_cols` are ints or CUDA int32 words
    (the reference uses seed and seed ^ 0x5bd1e995).  With `gw_out` (fp32 [N, K]) the weight
    gradient is accumulated into it in place -- gradient accumulation over microbatches -- and
    returned; otherwise a new tensor of `wgrad_dtype` is returned.  `sr_mode` picks the stochastic
    rounding (default: the module default of `nvq`); `overwrite` stores into `gw_out` instead of adding.
    `qxt`: the transposed operand of x from `linear_fwd(..., keep_xt=True)`; x may then be None.
    `am_gy`: amax(gy) if the caller already has it; `am_out`: else a zeroed device word to compute it into.
    `wgrad_stream`: the weight-gradient GEMM is off the backward's critical chain (nothing downstream reads dW before
    the optimizer), so it may run on this side stream beside the dgrad GEMM and whatever follows it: its CTAs fill
    the SMs the other kernels' last waves leave idle.  The caller joins the stream before it reads `gw_out` and
    passes a list as `keep_alive`, which receives the operands the side stream still reads (drop them after the join).
    `gw_owners`: data-parallel reduce-scatter in the weight-gradient GEMM's epilogue: the addresses of `gw_out` on every
    rank; the product is added into the row slab each rank owns (`nvq.mm(owners=)`; `overwrite` is then ignored: the
    caller clears the slabs once per step)."""
    gy = gy.contiguous()
    ag = am_gy if am_gy is not None else (nvq.amax(gy) if am_out is None else nvq.amax(gy, out=am_out, clear=False))
    if _tileable(gy):
        # both operands of gy from one pass over it
        qg, qgt = nvq.quant_rows_cols_rht(gy, signs, sr=True, seed=seed, seed_cols=seed_cols, am=ag, sr_mode=sr_mode)
    else:
        qg = nvq.quant_rows(gy, sr=True, seed=seed, am=ag, sr_mode=sr_mode)
        qgt = nvq.quant_cols_rht(gy, signs, sr=True, seed=seed_cols, am=ag, sr_mode=sr_mode)
    side = wgrad_stream if (gw_out is not None and wgrad_stream is not None) else None
    if side is not None:
        # the side stream starts from the quantized operands, not from the dgrad GEMM enqueued next
        if qxt is None:
            qxt = nvq.quant_cols_rht(x, signs, am=am_x)
        side.wait_stream(torch.cuda.current_stream())
    # dgrad: gx = gy @ w     (quantized along N; W^T uses the same 2D-block values)
    gx = nvq.mm(qg, qwt)
    # wgrad: gw = gy^T @ x   (both quantized along tokens, after a 16-pt RHT)
    if qxt is None:
        qxt = nvq.quant_cols_rht(x, signs, am=am_x)
    if side is not None:
        with torch.cuda.stream(side):
            gw = nvq.mm(qgt, qxt, out_dtype=torch.float32, out=gw_out, accumulate=not overwrite, splitk=0, owners=gw_owners)
        keep_alive.append((qgt, qxt))
    elif gw_out is not None:
        gw = nvq.mm(qgt, qxt, out_dtype=torch.float32, out=gw_out, accumulate=not overwrite, splitk=0, owners=gw_owners)
    else:
        gw = nvq.mm(qgt, qxt, out_dtype=wgrad_dtype)
    return gx, gw


class FP4LinearFn(torch.autograd.Function):
    """x [T, K] bf16, w [N, K] bf16 -> y [T, N] bf16 (llm-1b/model.py:45-69)."""

    @staticmethod
    def forward(ctx, x, w, lid, cache=None):
        qw = cache.q if cache is not None else nvq.quant_w2d(w, want=(True, False))[0]
        # the backward pass needs x only as the transposed RHT operand: keep that (0.56 byte per
        # element) instead of x
        y, am, qxt = linear_fwd(x, qw, keep_xt=True)
        ctx.save_for_backward(w, am, qxt.d, qxt.s, qxt.gs)
        ctx.lid, ctx.cache = lid, cache
        return y

    @staticmethod
    def backward(ctx, gy):
        w, am, xd, xs, xg = ctx.saved_tensors
        seed = sr_seed(ctx.lid)
        qwt = ctx.cache.qt if ctx.cache is not None else nvq.quant_w2d(w, want=(False, True))[1]
        gx, gw = linear_bwd(None, am, gy, qwt, seed, seed ^ 0x5bd1e995, wgrad_dtype=LinCtx.wgrad_dtype,
                            qxt=nvq.Q(xd, xs, xg))
        return gx, gw, None, None


class Linear(nn.Module):
    """Bias-free linear whose GEMMs run in NVFP4 when LinCtx.fp4, else BF16 (llm-1b/model.py:72-90)."""
    _next_id = 0

    def __init__(self, fin, fout, std, cache_weights=False):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(fout, fin))
        nn.init.trunc_normal_(self.weight, std=std, a=-3 * std, b=3 * std)
        self.lid = Linear._next_id
        Linear._next_id += 1
        self.cache = WeightCache(self.weight) if cache_weights else None

    def refresh(self):
        if self.cache is not None:
            self.cache.refresh()

    def forward(self, x):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        if LinCtx.fp4:
            if self.cache is not None and self.cache.q is None:
                self.cache.refresh()
            y = FP4LinearFn.apply(x2, self.weight, self.lid, self.cache)
        else:
            y = x2 @ self.weight.t()
        return y.view(*shp[:-1], -1)
