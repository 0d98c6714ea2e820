"""Torch (CPU, multi-threaded) restatement of the reference's fake-quant linear layer.
TEST / BASELINE INFRASTRUCTURE ONLY -- the product never imports it.

It follows small-model/model_ref.py (`fp4_round` :19-32, `e4m3` :35-36, `nvfp4_1d` :39-47,
`nvfp4_2d` :50-58, `_FP4Linear` :68-91) with the kernel contract of llm-1b/nvq.cu for the
wgrad operands (butterfly RHT16, scale from 4*amax, :136-152).  It exists because the reference
checkout is not available where the benchmark runs: `bench.py` times it on the host cores as the
CPU baseline.  Pinned like the numpy oracle: tests/test_oracle_golden.py compares it bit-for-bit
with the same model_ref fixtures.  Stochastic rounding here draws `torch.rand` like model_ref does
(timing and statistics only; the bit-level SR contract lives in nvfp4_oracle.py).
"""
import torch

_BOUNDS = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
_GRID = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def fp4_round(y, stochastic=False):
    """Nearest (ties to even code) or stochastic E2M1 value of y (model_ref.py:19-32)."""
    a = y.abs().clamp(max=6.0)
    if stochastic:
        step = torch.where(a < 2, 0.5, torch.where(a < 4, 1.0, 2.0))
        lo = torch.floor(a / step) * step
        up = torch.rand_like(a) < (a - lo) / step
        q = torch.where(up, lo + step, lo).clamp(max=6.0)
    else:
        # right=False: a == bound stays below the bound; ties then go up only at odd lower codes
        idx = torch.bucketize(a.contiguous(), _BOUNDS, right=False)
        tie_up = (a == 0.75) | (a == 1.75) | (a == 3.5)
        q = _GRID[idx + tie_up.long()]
    return torch.copysign(q, y)


def e4m3(x):
    return x.clamp(max=448.0).to(torch.float8_e4m3fn).float()


def nvfp4_1d(x, stochastic=False, gamax=None):
    """Quantize-dequantize along the last dim in blocks of 16 (model_ref.py:39-47)."""
    xf = x.float()
    amax = xf.abs().max() if gamax is None else gamax
    gs = (amax / 2688.0).clamp(min=1e-30)
    xb = xf.reshape(*xf.shape[:-1], -1, 16) / gs
    bs = e4m3(xb.abs().amax(-1, keepdim=True) / 6.0)
    q = fp4_round(xb / bs.clamp(min=1e-30), stochastic) * bs
    return (q * gs).reshape(xf.shape)


def nvfp4_2d(w):
    """16x16 block quantization for weights [out, in] (model_ref.py:50-58)."""
    wf = w.float()
    o, i = wf.shape
    gs = (wf.abs().max() / 2688.0).clamp(min=1e-30)
    wb = wf.reshape(o // 16, 16, i // 16, 16).permute(0, 2, 1, 3) / gs
    bs = e4m3(wb.abs().amax((-1, -2), keepdim=True) / 6.0)
    q = fp4_round(wb / bs.clamp(min=1e-30)) * bs
    return (q * gs).permute(0, 2, 1, 3).reshape(o, i)


def rht16_t(x, signs):
    """x [M, C] -> RHT16 along M of x^T, [C, M]: sign flip, butterflies h = 1,2,4,8, x0.25
    (llm-1b/nvq.cu:136-152)."""
    M, C = x.shape
    v = x.float().t().reshape(C, M // 16, 16)
    sv = torch.tensor([-1.0 if (signs >> i) & 1 else 1.0 for i in range(16)])
    v = v * sv
    for h in (1, 2, 4, 8):
        v = v.reshape(C, M // 16, 16 // (2 * h), 2, h)
        a, b = v[..., 0, :], v[..., 1, :]
        v = torch.stack([a + b, a - b], dim=-2).reshape(C, M // 16, 16)
    return (v * 0.25).reshape(C, M)


def linear_fwd_bwd(x, wq, gy, signs, stochastic=True):
    """fprop / dgrad / wgrad of llm-1b/model.py:45-69 on dequantized operands, `wq` = nvfp4_2d(w)."""
    y = nvfp4_1d(x) @ wq.t()
    ag = gy.float().abs().max()
    gx = nvfp4_1d(gy, stochastic, gamax=ag) @ wq
    gt = nvfp4_1d(rht16_t(gy, signs), stochastic, gamax=ag * 4)
    xt = nvfp4_1d(rht16_t(x, signs), gamax=x.float().abs().max() * 4)
    return y, gx, gt @ xt.t()
