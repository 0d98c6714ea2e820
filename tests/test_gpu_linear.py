"""GPU parity of the autograd NVFP4 linear layer (llm-1b/model.py:45-69 recipe) with the oracle's
whole-layer restatement, on a shape small enough for the CPU to finish in seconds."""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from tests.gpu_util import make_dy, make_w, make_x, rel_fro, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cache", [False, True])
def test_linear_fwd_bwd_matches_oracle(cache):
    from nvfp4_training_b200 import _lib
    from nvfp4_training_b200.linear import FP4LinearFn, LinCtx, WeightCache, _RHT_SIGNS, sr_seed
    T, K, N = 512, 256, 384
    x, w, gy = make_x(1, T, K), make_w(2, N, K), make_dy(3, T, N)
    LinCtx.seed, LinCtx.wgrad_dtype = 12, torch.float32
    lid = 3
    xd = to_dev(x).requires_grad_(True)
    wd = to_dev(w).requires_grad_(True)
    wc = WeightCache(wd).refresh() if cache else None
    y = FP4LinearFn.apply(xd, wd, lid, wc)
    y.backward(to_dev(gy))
    seed = sr_seed(lid)
    assert seed == (12 * 1000003 + 3 * 7919) & 0xFFFFFFFF
    ry, rgx, rgw = O.linear_fwd_bwd(x, w, gy, _RHT_SIGNS, seed=seed, sr_mode=O.SR_DITHER_NVQ)
    # same codes/scales on both sides, so only accumulation order and the bf16 output cast differ
    assert rel_fro(y.detach().float().cpu().numpy(), ry) <= 4e-3
    assert rel_fro(xd.grad.float().cpu().numpy(), rgx) <= 4e-3
    assert wd.grad.dtype == torch.float32 or wd.grad.dtype == torch.bfloat16
    assert rel_fro(wd.grad.float().cpu().numpy(), rgw) <= 4e-3
    # and the quantized layer tracks the exact one within FP4 noise
    assert rel_fro(ry, x @ w.T) < 0.15
    _lib.check_status()
    LinCtx.wgrad_dtype = torch.bfloat16


def test_linear_module_bf16_switch():
    from nvfp4_training_b200.linear import Linear, LinCtx
    torch.manual_seed(0)
    lin = Linear(256, 384, std=0.02).cuda().bfloat16()
    x = torch.randn(2, 64, 256, device="cuda", dtype=torch.bfloat16)
    LinCtx.fp4 = True
    y4 = lin(x)
    LinCtx.fp4 = False
    y16 = lin(x)
    LinCtx.fp4 = True
    assert y4.shape == (2, 64, 384)
    assert ((y4.float() - y16.float()).norm() / y16.float().norm()).item() < 0.2


def test_fp4torch_custom_op_linear():
    """small-model/fp4torch.py flavour: nvfp4::linear with autograd, weights quantized once by
    FP4Weight; forward equals the dequant matmul, gradients track the exact ones within FP4 noise."""
    from nvfp4_training_b200 import _lib, fp4ops, fp4torch
    torch.manual_seed(0)
    T, K, N = 256, 256, 384
    x = torch.randn(2, T // 2, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).requires_grad_(True)
    fw = fp4torch.FP4Weight(w)
    y = torch.ops.nvfp4.linear(x, w, fw.wd, fw.ws, fw.wtd, fw.wts, fw.amax)
    assert y.shape == (2, T // 2, N) and y.dtype == torch.bfloat16
    qx = fp4ops.quant_rows(x.detach().reshape(-1, K))
    ref = fp4ops.dequant(qx) @ fp4ops.dequant(fp4ops.Q(fw.wd, fw.ws, fw.amax)).t()
    assert ((y.float().reshape(-1, N) - ref).norm() / ref.norm()).item() <= 4e-3
    g = torch.randn_like(y) * 1e-3
    y.backward(g)
    ex_dx = g.float().reshape(-1, N) @ w.detach()
    ex_dw = g.float().reshape(-1, N).t() @ x.detach().float().reshape(-1, K)
    assert w.grad.dtype == torch.float32 and w.grad.shape == (N, K)
    assert ((x.grad.float().reshape(-1, K) - ex_dx).norm() / ex_dx.norm()).item() < 0.2
    assert ((w.grad - ex_dw).norm() / ex_dw.norm()).item() < 0.25
    fw.refresh()
    _lib.check_status()


def test_fp4weight_keeps_swizzled_scales():
    """FP4Weight holds the swizzled form of its scales and `fp4ops.gemm` finds it by the address of the row-major
    scales the custom ops pass: same bytes out as the path that swizzles both operands per call, also after a
    refresh with new weight values (the copies are rewritten with the weight)."""
    from nvfp4_training_b200 import _lib, fp4ops, fp4torch
    torch.manual_seed(3)
    T, K, N = 256, 256, 384
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda") / K ** 0.5
    fw = fp4torch.FP4Weight(w)
    for rnd in range(2):
        assert fp4ops.swizzled_of(fw.ws) is not None and fp4ops.swizzled_of(fw.wts) is not None
        assert torch.equal(fp4ops.swizzled_of(fw.ws), fp4ops.swizzle_scales(fw.ws))
        assert torch.equal(fp4ops.swizzled_of(fw.wts), fp4ops.swizzle_scales(fw.wts))
        y = torch.ops.nvfp4.fwd(x, fw.wd, fw.ws, fw.amax)
        # the same operands through copies nobody has registered: both scales swizzled inside the call
        y_plain = fp4ops.gemm(fp4ops.quant_rows(x), fp4ops.Q(fw.wd.clone(), fw.ws.clone(), fw.amax))
        assert torch.equal(y, y_plain)
        g = torch.randn(T, N, device="cuda", dtype=torch.bfloat16)
        qg = fp4ops.quant_rows(g)
        dx = fp4ops.gemm(qg, fp4ops.Q(fw.wtd, fw.wts, fw.amax))
        assert torch.equal(dx, fp4ops.gemm(qg, fp4ops.Q(fw.wtd.clone(), fw.wts.clone(), fw.amax)))
        w.mul_(1.7).add_(torch.randn_like(w) * 0.01)
        fw.refresh()
    _lib.check_status()
