"""Drop-in proof through the reference's callers: after `install_as_reference_modules()` the names
`nvq` and `fp4ops` resolve to this package, and the call sequences of the reference's two layer
implementations run against them exactly as the reference makes them --

  * `FP4LinearFn` of llm-1b/model.py:45-69: `import nvq`; forward `quant_rows(x)`, `quant_w2d(w)` (both
    halves returned, one used), `mm(qx, qw)`; backward `amax(gy)`, `quant_w2d(w)` again, `quant_rows(gy,
    sr=True, seed=, am=)`, `quant_cols_rht(gy, signs, sr=True, seed=, am=)`, `quant_cols_rht(x, signs)` and
    bf16 `mm` for both gradients; x and w saved as bf16 tensors;
  * `fp4_fwd` / `fp4_bwd` of small-model/fp4torch.py:19-38: `import fp4ops as F`; `F.gemm(F.quant_rows(x2),
    F.Q(wd, ws, wamax))`, `F.gemm(F.quant_rows(g2, sr=True, seed=), F.Q(wtd, wts, wamax))`,
    `F.gemm(F.quant_cols_rht(g2, signs, sr=True, seed=), F.quant_cols_rht(x2, signs), splitk=16)` on
    weights from `F.quant_w2d(fp32 w)`.

Both are compared with the oracle's whole-layer restatement on the same seeds (bf16 outputs: relative
Frobenius error <= 4e-3; FP32 split-K wgrad: <= 1e-4)."""
import importlib

import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from tests.gpu_util import make_dy, make_w, make_x, rel_fro, to_dev

pytestmark = pytest.mark.gpu

SIGNS = 0b1010011010110001          # llm-1b/model.py:42


def test_reference_autograd_function_on_import_nvq():
    import nvfp4_training_b200
    from nvfp4_training_b200 import _lib
    nvfp4_training_b200.install_as_reference_modules()
    nvq = importlib.import_module("nvq")                     # what the reference's `import nvq` resolves to
    assert nvq.__name__ == "nvfp4_training_b200.nvq"
    micro_seed, lid = 4, 6

    class Fn(torch.autograd.Function):                       # call sequence of llm-1b/model.py:45-69
        @staticmethod
        def forward(ctx, x, w):
            ctx.save_for_backward(x, w)
            qx = nvq.quant_rows(x)
            qw, _ = nvq.quant_w2d(w)
            return nvq.mm(qx, qw)

        @staticmethod
        def backward(ctx, gy):
            x, w = ctx.saved_tensors
            gy = gy.contiguous()
            seed = (micro_seed * 1000003 + lid * 7919) & 0xFFFFFFFF
            ag = nvq.amax(gy)
            _, qwt = nvq.quant_w2d(w)
            qg = nvq.quant_rows(gy, sr=True, seed=seed, am=ag)
            gx = nvq.mm(qg, qwt)
            qgt = nvq.quant_cols_rht(gy, SIGNS, sr=True, seed=seed ^ 0x5bd1e995, am=ag)
            qxt = nvq.quant_cols_rht(x, SIGNS)
            return gx, nvq.mm(qgt, qxt)

    T, K, N = 512, 384, 640
    x, w, gy = make_x(1, T, K), make_w(2, N, K), make_dy(3, T, N)
    xd, wd = to_dev(x).requires_grad_(True), to_dev(w).requires_grad_(True)
    y = Fn.apply(xd, wd)
    y.backward(to_dev(gy))
    assert y.dtype == torch.bfloat16 and wd.grad.dtype == torch.bfloat16 and wd.grad.shape == (N, K)
    seed = (micro_seed * 1000003 + lid * 7919) & 0xFFFFFFFF
    ry, rgx, rgw = O.linear_fwd_bwd(x, w, gy, SIGNS, seed=seed, sr_mode=O.SR_DITHER_NVQ)
    assert rel_fro(y.detach().float().cpu().numpy(), ry) <= 4e-3
    assert rel_fro(xd.grad.float().cpu().numpy(), rgx) <= 4e-3
    assert rel_fro(wd.grad.float().cpu().numpy(), rgw) <= 4e-3
    _lib.check_status()


def test_reference_custom_op_bodies_on_import_fp4ops():
    import nvfp4_training_b200
    from nvfp4_training_b200 import _lib
    nvfp4_training_b200.install_as_reference_modules()
    F = importlib.import_module("fp4ops")                    # `import fp4ops as F`
    assert F.__name__ == "nvfp4_training_b200.fp4ops"
    T, K, N = 512, 256, 384
    x, gy = make_x(4, T, K), make_dy(5, T, N)
    w = np.random.default_rng(6).standard_normal((N, K)).astype(np.float32) * 0.02      # FP32 master weight
    q, qt = F.quant_w2d(torch.from_numpy(w).cuda())
    wd, ws, wtd, wts, wamax = q.d, q.s, qt.d, qt.s, q.amax
    xg, gg = to_dev(x).reshape(2, T // 2, K), to_dev(gy).reshape(2, T // 2, N)
    # fp4_fwd (small-model/fp4torch.py:19-23)
    x2 = xg.reshape(-1, xg.shape[-1])
    y = F.gemm(F.quant_rows(x2), F.Q(wd, ws, wamax)).reshape(*xg.shape[:-1], wd.shape[0])
    # fp4_bwd (small-model/fp4torch.py:31-38)
    g2 = gg.reshape(-1, gg.shape[-1]).contiguous()
    x2 = xg.reshape(-1, xg.shape[-1]).contiguous()
    s1, s2, signs = 2654435761 & 0xFFFFFFFF, (2 * 2654435761) & 0xFFFFFFFF, 0x3C5A
    dx = F.gemm(F.quant_rows(g2, sr=True, seed=s1), F.Q(wtd, wts, wamax)).reshape(xg.shape)
    dw = F.gemm(F.quant_cols_rht(g2, signs, sr=True, seed=s2), F.quant_cols_rht(x2, signs), splitk=16)
    assert y.dtype == torch.bfloat16 and dx.dtype == torch.bfloat16 and dw.dtype == torch.float32
    # oracle with the fp4k streams (element-indexed hashing, llm-1b/fp4k.cu:53-58)
    oq, os_, oqt, ost, ogs = O.quant_w2d(w)
    a = O.quant_rows(x)
    ry = O.gemm_dequant(a[0], a[1], a[2], oq, os_, ogs)
    g = O.quant_rows(gy, sr_mode=O.SR_DITHER_FP4K, seed=s1)
    rdx = O.gemm_dequant(g[0], g[1], g[2], oqt, ost, ogs)
    gt = O.quant_cols_rht(gy, signs, sr_mode=O.SR_DITHER_FP4K, seed=s2)
    xt = O.quant_cols_rht(x, signs)
    rdw = O.gemm_dequant(gt[0], gt[1], gt[2], xt[0], xt[1], xt[2])
    assert rel_fro(y.float().cpu().numpy().reshape(T, N), ry) <= 4e-3
    assert rel_fro(dx.float().cpu().numpy().reshape(T, K), rdx) <= 4e-3
    assert rel_fro(dw.cpu().numpy(), rdw) <= 1e-4
    _lib.check_status()
