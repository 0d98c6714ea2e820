"""The NVFP4 linear layer behind torch custom ops, i.e. the surface small-model/fp4torch.py gives a
compiled model: `torch.ops.nvfp4.fwd`, `.bwd`, `.linear` (with autograd) and `FP4Weight`.

Recipe (small-model/fp4torch.py:19-38):  y = Q_rn(x) @ Q2d(W)^T;  dx = Q_sr(dy) @ Q2d(W);
dW = Q_sr(H dy)^T @ Q_rn(H x) accumulated in FP32 with split-K 16.  Here the two operands of dy come
from one pass over dy when its shape allows (`fp4ops.quant_rows_cols_rht`), and `FP4Weight.refresh`
rewrites its buffers in place instead of copying into them.

Randomness follows the reference: stochastic-rounding seeds are a process-wide counter times
2654435761, the 16 Hadamard sign bits come from Python's `random` once per backward call.
"""
import itertools
import random

import torch

from . import fp4ops as F

_LIB = torch.library.Library("nvfp4", "DEF")
_LIB.define("fwd(Tensor x, Tensor wd, Tensor ws, Tensor wamax) -> Tensor")
_LIB.define("bwd(Tensor g, Tensor x, Tensor wtd, Tensor wts, Tensor wamax) -> (Tensor, Tensor)")
_LIB.define("linear(Tensor x, Tensor w, Tensor wd, Tensor ws, Tensor wtd, Tensor wts, Tensor wamax) -> Tensor")

_calls = itertools.count(1)


def _next_seed():
    return (next(_calls) * 2654435761) & 0xFFFFFFFF


def _rows(t):
    """[..., C] -> contiguous [R, C]."""
    return t.reshape(-1, t.shape[-1]).contiguous()


def _fprop(x, wd, ws, wamax):
    y = F.gemm(F.quant_rows(_rows(x)), F.Q(wd, ws, wamax))
    return y.reshape(*x.shape[:-1], wd.shape[0])


def _grads(g, x, wtd, wts, wamax):
    g2, x2 = _rows(g), _rows(x)
    signs = random.getrandbits(16)
    seed_rows, seed_cols = _next_seed(), _next_seed()
    if g2.shape[0] % 128 == 0 and g2.shape[1] % 64 == 0:
        qg, qgt = F.quant_rows_cols_rht(g2, signs, sr=True, seed=seed_rows, seed_cols=seed_cols)
    else:
        qg = F.quant_rows(g2, sr=True, seed=seed_rows)
        qgt = F.quant_cols_rht(g2, signs, sr=True, seed=seed_cols)
    dx = F.gemm(qg, F.Q(wtd, wts, wamax)).reshape(x.shape)
    dw = F.gemm(qgt, F.quant_cols_rht(x2, signs), splitk=16)
    return dx, dw


torch.library.impl(_LIB, "fwd", "CUDA")(_fprop)
torch.library.impl(_LIB, "bwd", "CUDA")(_grads)
torch.library.impl(_LIB, "linear", "CUDA")(lambda x, w, wd, ws, wtd, wts, wamax: _fprop(x, wd, ws, wamax))

torch.library.register_fake("nvfp4::fwd")(lambda x, wd, ws, wamax: x.new_empty(*x.shape[:-1], wd.shape[0]))
torch.library.register_fake("nvfp4::bwd")(
    lambda g, x, wtd, wts, wamax: (x.new_empty(x.shape), g.new_empty(g.shape[-1], x.shape[-1], dtype=torch.float32)))
torch.library.register_fake("nvfp4::linear")(
    lambda x, w, wd, ws, wtd, wts, wamax: x.new_empty(*x.shape[:-1], w.shape[0]))

fp4_fwd, fp4_bwd, fp4_linear = torch.ops.nvfp4.fwd, torch.ops.nvfp4.bwd, torch.ops.nvfp4.linear


def _save(ctx, inputs, output):
    x, _w, _wd, _ws, wtd, wts, wamax = inputs
    ctx.save_for_backward(x, wtd, wts, wamax)


def _linear_backward(ctx, g):
    dx, dw = fp4_bwd(g.contiguous(), *ctx.saved_tensors)
    return (dx, dw) + (None,) * 5


torch.library.register_autograd("nvfp4::linear", _linear_backward, setup_context=_save)


class FP4Weight:
    """Quantized copies of an FP32 master weight and of its transpose, refreshed once per optimizer
    step (small-model/fp4torch.py:71-84).  Attributes: wd, ws (W), wtd, wts (W^T), amax."""

    def __init__(self, w):
        self.w = w
        self._q = None
        self.refresh()

    @torch.no_grad()
    def refresh(self):
        self._q = F.quant_w2d(self.w.data, out=self._q)      # in place after the first call
        qw, qwt = self._q
        self.wd, self.ws, self.wtd, self.wts, self.amax = qw.d, qw.s, qwt.d, qwt.s, qw.amax
        # the tensor core reads swizzled scales: keep those of the weight (they change only here), so that each
        # GEMM swizzles just its activation operand
        N, K = self.w.shape
        if qw.sw is None and N % 128 == 0 and K % 128 == 0:     # later refreshes rewrite them inside quant_w2d
            qw.sw, qwt.sw = F.swizzle_scales(qw.s), F.swizzle_scales(qwt.s)
            F.remember_swizzled(qw.s, qw.sw)
            F.remember_swizzled(qwt.s, qwt.sw)
        return self
