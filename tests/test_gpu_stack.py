"""GPU check of `LinearStack`, the data-parallel workload the benchmark times: a tiny architecture
(2 blocks + head, d = 256) run for one step of two microbatches

  * with CUDA graphs and without: the FP32 weight gradients must be bit-equal (the first microbatch
    stores dW, the second adds once, so the order of operations is fixed), which covers capture and
    replay, the device-side stochastic-rounding seeds, the `overwrite=first` path, the flat per-block
    gradient buffers and the weight-refresh graph;
  * against the oracle's whole-layer restatement with the same seeds (hardware stochastic rounding
    model), summed over the two microbatches: relative Frobenius error <= 1e-4 for FP32 dW, <= 4e-3
    for the bf16 y and dX of one eager block pass.
"""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from tests.gpu_util import rel_fro

pytestmark = pytest.mark.gpu


def f32(t):
    return t.float().cpu().numpy()


def tiny_stack(use_graphs, seed=3):
    from nvfp4_training_b200.stack import LinearStack, StackConfig
    cfg = StackConfig(vocab=512, d=256, layers=2, heads=2, kv_heads=1, ff=384, lm_head=True)
    st = LinearStack(cfg, 256, torch.device("cuda"), seed=seed, use_graphs=use_graphs)
    if use_graphs:
        st.capture()
    return st


def test_stack_graphs_equal_eager_and_oracle():
    from nvfp4_training_b200 import _lib
    from nvfp4_training_b200.linear import _RHT_SIGNS
    a, b = tiny_stack(True), tiny_stack(False)
    assert a.graphs_fwd is not None and b.graphs_fwd is None
    for pa, pb in zip([p for blk in a.blocks for p in blk], [p for blk in b.blocks for p in blk]):
        assert torch.equal(pa.w, pb.w)
    first_micro = a.micro_count
    assert first_micro == b.micro_count
    for st in (a, b):
        st.step(2, do_allreduce=False)
    torch.cuda.synchronize()
    _lib.check_status()
    for pa, pb in zip([p for blk in a.blocks for p in blk], [p for blk in b.blocks for p in blk]):
        assert torch.equal(pa.gw, pb.gw), pa.name
        assert pa.gw.abs().max().item() > 0
    # a second step replays the same graphs with new seeds: still equal, and different from the first
    g0 = a.blocks[0][2].gw.clone()
    for st in (a, b):
        st.step(2, do_allreduce=False)
    torch.cuda.synchronize()
    for pa, pb in zip([p for blk in a.blocks for p in blk], [p for blk in b.blocks for p in blk]):
        assert torch.equal(pa.gw, pb.gw), pa.name
    assert not torch.equal(g0, a.blocks[0][2].gw)

    # oracle: dW of three projections over the two microbatches of the FIRST step of a fresh stack
    c = tiny_stack(True)
    c.step(2, do_allreduce=False)
    torch.cuda.synchronize()
    for p in (c.blocks[0][0], c.blocks[1][3], c.blocks[2][0]):
        x, w, gy = f32(c.x_pool[p.name]), f32(p.w), f32(c.gy_pool[p.name])
        want = 0.0
        for m in (first_micro, first_micro + 1):
            seed = (p.lid * 7919 + m * 1000003) & 0xFFFFFFFF
            _, _, gw = O.linear_fwd_bwd(x, w, gy, _RHT_SIGNS, seed=seed, sr_mode=O.SR_HW)
            want = want + gw.astype(np.float64)
        assert rel_fro(f32(p.gw), want) <= 1e-4, (p.name, rel_fro(f32(p.gw), want))
    # y and dX of one eager block pass with the seeds now in device memory
    projs = b.blocks[1]
    b._fwd_block(projs, keep=True)
    b._bwd_block(projs, keep=True, first=True)
    torch.cuda.synchronize()
    seeds = b.seeds.cpu().numpy().astype(np.int64) & 0xFFFFFFFF
    for p in projs:
        x, w, gy = f32(b.x_pool[p.name]), f32(p.w), f32(b.gy_pool[p.name])
        assert int(seeds[p.lid, 1]) == int(seeds[p.lid, 0]) ^ 0x5BD1E995
        y, gx, gw = O.linear_fwd_bwd(x, w, gy, _RHT_SIGNS, seed=int(seeds[p.lid, 0]), sr_mode=O.SR_HW)
        assert rel_fro(f32(p.y), y) <= 4e-3 and rel_fro(f32(p.gx), gx) <= 4e-3, p.name
        assert rel_fro(f32(p.gw), gw) <= 1e-4, p.name
    _lib.check_status()


def test_stack_separate_weight_and_input_seeds():
    """Ranks of a data-parallel job share the weight seed and differ in the input seed: same weights,
    different activations."""
    from nvfp4_training_b200.stack import LinearStack, StackConfig
    cfg = StackConfig(vocab=512, d=256, layers=1, heads=2, kv_heads=1, ff=384, lm_head=False)
    a = LinearStack(cfg, 128, torch.device("cuda"), seed=0, input_seed=10, use_graphs=False)
    b = LinearStack(cfg, 128, torch.device("cuda"), seed=0, input_seed=11, use_graphs=False)
    for pa, pb in zip(a.blocks[0], b.blocks[0]):
        assert torch.equal(pa.w, pb.w)
    assert not torch.equal(a.x_pool["qkv"], b.x_pool["qkv"])


def test_stack_emitter_mode_graphs_equal_eager_and_oracle():
    """The emitter mode of the stack (row operands with per-row scales, column operands with delayed scales,
    scales applied in the GEMM epilogues): graph replay equals eager bit for bit, the delayed amax settles at
    margin x observed, and dW of one projection equals the oracle's restatement of the emitters (FP64 product of the
    dequantized operands) within 1e-4."""
    from nvfp4_training_b200 import _lib
    from nvfp4_training_b200.linear import _RHT_SIGNS
    from nvfp4_training_b200.stack import EMIT_MARGIN, LinearStack, StackConfig
    cfg = StackConfig(vocab=512, d=256, layers=2, heads=2, kv_heads=1, ff=512, lm_head=True)
    a = LinearStack(cfg, 256, torch.device("cuda"), seed=3, use_graphs=True, mode="emit")
    a.capture()
    b = LinearStack(cfg, 256, torch.device("cuda"), seed=3, use_graphs=False, mode="emit")
    b.calibrate()
    assert torch.equal(a.amax_use, b.amax_use)
    for st in (a, b):
        st.step(2, do_allreduce=False)
    torch.cuda.synchronize()
    _lib.check_status()
    for pa, pb in zip([p for blk in a.blocks for p in blk], [p for blk in b.blocks for p in blk]):
        assert torch.equal(pa.gw, pb.gw), pa.name
        assert pa.gw.abs().max().item() > 0
    # oracle for one projection and ONE microbatch (eager, first = overwrite)
    p = b.blocks[0][2]
    x, gy = f32(b.x_pool[p.name]), f32(b.gy_pool[p.name])
    use = b.amax_use.cpu().numpy()
    obs_x = np.float32(np.abs(O.rht16_cols(x, _RHT_SIGNS)).max())
    assert use[p.lid, 0] == np.float32(obs_x * np.float32(EMIT_MARGIN))
    seed = int(b.rng[0].item())
    b._fwd_block(b.blocks[0], keep=True)
    b._bwd_block(b.blocks[0], keep=True, first=True)
    torch.cuda.synchronize()
    cx, sx, _ = O.emit_cols(x, _RHT_SIGNS, use[p.lid, 0])
    cg, sg, _ = O.emit_cols(gy, _RHT_SIGNS, use[p.lid, 1], seed=seed, sr="hw", salt=p.lid * 8 + 2)
    want = O.gemm_unit(cg, sg, cx, sx) * (float(use[p.lid, 1]) / 2688.0) * (float(use[p.lid, 0]) / 2688.0)
    assert rel_fro(f32(p.gw), want) <= 1e-4
    # forward y and dgrad of the same projection: per-row scales in the epilogue
    w = f32(p.w)
    rc, rsb, rs = O.emit_rows(x)
    wc, ws, wct, wst, wgs = O.quant_w2d(w)
    y = O.gemm_unit(rc, rsb, wc, ws) * rs.astype(np.float64)[:, None] * float(wgs)
    assert rel_fro(f32(p.y), y) <= 4e-3
    gc, gsb, grs = O.emit_rows(gy, seed=seed, sr="hw", salt=p.lid * 8 + 1)
    gx = O.gemm_unit(gc, gsb, wct, wst) * grs.astype(np.float64)[:, None] * float(wgs)
    assert rel_fro(f32(p.gx), gx) <= 4e-3
    _lib.check_status()


def test_stack_programmatic_launch_on_equals_off():
    """The kernels of a projection follow each other by programmatic dependent launch (each may start its set-up while
    its predecessor drains and waits for it before touching global memory).  Same seeds, the switch on and off, with
    graphs and without, weight gradients on a side stream or not: bit-equal FP32 weight gradients after two steps."""
    from nvfp4_training_b200 import _lib
    from nvfp4_training_b200.stack import LinearStack, StackConfig
    lib = _lib.load()
    cfg = StackConfig(vocab=512, d=256, layers=2, heads=2, kv_heads=1, ff=384, lm_head=True)
    grads = []
    try:
        for pdl, graphs, side in ((1, True, True), (0, True, True), (1, False, True), (1, True, False), (0, False, False)):
            assert lib.nvfp4_set_pdl(pdl) == 0
            st = LinearStack(cfg, 256, torch.device("cuda"), seed=5, use_graphs=graphs, wgrad_side_stream=side)
            if graphs:
                st.capture()
            for _ in range(2):
                st.step(2, do_allreduce=False)
            torch.cuda.synchronize()
            grads.append([p.gw.clone() for blk in st.blocks for p in blk])
    finally:
        lib.nvfp4_set_pdl(1)
    _lib.check_status()
    for other in grads[1:]:
        for g0, g1 in zip(grads[0], other):
            assert torch.equal(g0, g1)
    assert grads[0][0].abs().max().item() > 0


def test_amax_update_keeps_the_larger_value():
    from nvfp4_training_b200 import nvq
    torch.manual_seed(0)
    x = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16)
    words = torch.zeros(3, device="cuda")
    nvq.amax(x, out=words[0:1], clear=False)
    nvq.amax(x * 4, out=words[1:2], clear=False)
    nvq.amax(x, out=words[1:2], clear=False)           # smaller: leaves the word
    assert words[0].item() == x.abs().max().item()
    assert words[1].item() == (x * 4).abs().max().item()
    assert words[2].item() == 0.0
    assert nvq.amax(x).item() == words[0].item()


def test_stack_weights_requantized_behind_the_backward_pass():
    """`overlap_refresh`: a block's weights are re-quantized on the side stream right after the block's backward (and
    all-reduce), after the `after_reduce` hook where a trainer updates them, instead of all at the start of the next
    step.  With a hook that changes the weights every step, after three steps the quantized weights give the same
    forward output as those of a stack that re-quantizes everything at the start of each step (so the overlapped
    refresh saw the updated weights), bit for bit, with graphs and without; the gradients agree as well."""
    from nvfp4_training_b200 import _lib
    from nvfp4_training_b200.stack import LinearStack, StackConfig
    cfg = StackConfig(vocab=512, d=256, layers=2, heads=2, kv_heads=1, ff=384, lm_head=True)

    def update(b, projs):
        for p in projs:
            p.w.mul_(1.25)           # stands for the block's optimizer update

    grads, outs = [], []
    for overlap, graphs in ((True, True), (False, True), (True, False), (False, False)):
        st = LinearStack(cfg, 256, torch.device("cuda"), seed=7, use_graphs=graphs, overlap_refresh=overlap)
        st.after_reduce = update
        if graphs:
            st.capture()
        out = []
        for _ in range(3):
            st.step(2, do_allreduce=False)
            torch.cuda.synchronize()
            out.append([p.gw.clone() for blk in st.blocks for p in blk])
        grads.append(out)
        if not overlap:
            st.refresh_weights()     # what the next step would start with
        for projs in st.blocks:
            st._fwd_block(projs, keep=True)
        torch.cuda.synchronize()
        outs.append([p.y.clone() for blk in st.blocks for p in blk])
    _lib.check_status()
    for other in outs[1:]:
        for y0, y1 in zip(outs[0], other):
            assert torch.equal(y0, y1)
    assert outs[0][0].abs().max().item() > 0
    for other in grads[1:]:
        for s0, s1 in zip(grads[0], other):
            for g0, g1 in zip(s0, s1):
                assert torch.equal(g0, g1)
