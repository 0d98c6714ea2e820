"""Benchmark of the NVFP4 linear-layer hot path on B200.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torch.distributed.run)
    python bench.py --impl reference --steps K --warmup W     (the reference's CPU torch path, host cores)

Workload (both arms): every NVFP4 linear of the 1.0B architecture -- 20 blocks x {qkv, o, gate/up,
down} + the 49,152-row LM head -- forward and backward (fprop, dgrad, wgrad with RHT16 and stochastic
rounding), global batch 32 x 2048 tokens sharded by rows over N GPUs with replicated random-init
weights, FP32 weight gradients all-reduced with NCCL.  A step re-quantizes all weights once, clears
dW, runs the rank's microbatches and the all-reduce.  Metric: tokens/s of the whole job.

Rank 0 prints ONE JSON line.  Extra keys: `roofline` (the GEMM, timed alone with CUDA events),
`cpu_baseline` (the torch restatement of the reference on a bounded sample, N = 1 only), `e2e`
(same step with the batch copied from pinned host memory and a result read back every step),
`detail` (per-kernel-class numbers).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GLOBAL_TOKENS = 32 * 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """nvidia-smi sampling of SM clock and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1])); power.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.unlink(self.path)
        if sm:
            busy = [s for s, p in zip(sm, power) if p > 0.5 * max(power)] or sm
            out.update(sm_mhz=statistics.median(busy), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm),
                       power_w_max=max(power))
        return out


# ------------------------------------------------------------------------------------------ reference arm (CPU)
def cpu_reference_sample(tokens, threads):
    """One bounded sample of the workload on the host: one block's four projections (weights
    re-quantized, `tokens` rows forward + backward) with the torch restatement of the reference.
    Returns (seconds for weight quantization, seconds for the token pass)."""
    import torch
    from oracle import torch_ref as T
    from nvfp4_training_b200.stack import StackConfig
    torch.set_num_threads(threads)
    cfg = StackConfig()
    g = torch.Generator().manual_seed(0)
    t_w = t_tok = 0.0
    for name, N, K, std in cfg.block_shapes():
        w = (torch.randn(N, K, generator=g) * std).bfloat16()
        x = torch.randn(tokens, K, generator=g).bfloat16()
        gy = (torch.randn(tokens, N, generator=g) * 1e-3).bfloat16()
        t0 = time.perf_counter()
        wq = T.nvfp4_2d(w)
        t1 = time.perf_counter()
        T.linear_fwd_bwd(x, wq, gy, 0b1010011010110001, stochastic=True)
        t2 = time.perf_counter()
        t_w += t1 - t0
        t_tok += t2 - t1
    return t_w, t_tok


def cpu_tokens_per_s(t_w, t_tok, tokens):
    """Extrapolate the one-block sample to the full step: weights of all 20 blocks + head once,
    65,536 tokens through all of them, scaled by parameter count and FLOPs."""
    from nvfp4_training_b200.stack import StackConfig
    cfg = StackConfig()
    block_params = sum(n * k for _, n, k, _ in cfg.block_shapes())
    scale = cfg.n_params() / block_params
    step_s = t_w * scale + t_tok * scale * (GLOBAL_TOKENS / tokens)
    return GLOBAL_TOKENS / step_s


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    tokens = 256
    for _ in range(max(args.warmup, 0) and 1):
        cpu_reference_sample(tokens, threads)
    vals = []
    t_all = time.perf_counter()
    for _ in range(max(1, args.steps)):
        t_w, t_tok = cpu_reference_sample(tokens, threads)
        vals.append(cpu_tokens_per_s(t_w, t_tok, tokens))
    dt = (time.perf_counter() - t_all) / max(1, args.steps)
    v = statistics.median(vals)
    sample = (f"one block (qkv,o,gate/up,down) weight quant + {tokens} tokens fwd+bwd per step with the torch "
              "restatement of small-model/model_ref.py, extrapolated to 20 blocks + LM head and 65,536 tokens "
              "by parameter count")
    print(json.dumps({
        "impl": "reference", "metric": "tokens/s", "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": GLOBAL_TOKENS / v * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp4(e2m1)+ue4m3 scales, fp32 math on CPU", "data": "synthetic",
        "config": workload_config(args.gpus, None, None),
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample,
                         "sample_seconds": dt},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(n_gpus, microbatch, n_micro):
    return {"workload": "NVFP4 linear fwd+bwd (fprop, dgrad, wgrad+RHT16, SR grads) of every linear of the 1.0B "
                        "architecture: 20 x {qkv 2048->3072, o 2048->2048, gate/up 2048->11264, down 5632->2048} + "
                        "LM head 2048->49152; weights re-quantized once per step; FP32 dW all-reduce",
            "global_batch_tokens": GLOBAL_TOKENS, "seq_len": 2048, "sequences": 32,
            "parallelism": f"dp{n_gpus} (token rows sharded, weights replicated)",
            "microbatch_tokens": microbatch, "microbatches_per_rank": n_micro,
            "l2": "per-step working set (2 GB bf16 weights, 1.1 GB packed weights, 4 GB dW, activations) >> 126 MB L2; "
                  "isolated-kernel timings rotate operand sets larger than L2"}


# ------------------------------------------------------------------------------------------ GPU arm
def time_events(fn, iters, warm=3):
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e-3


def time_graph(fn, iters, warm=2):
    """Like time_events, with the `iters` calls captured once into a CUDA graph and replayed: the timing then holds no
    host launch overhead (a Python call into the library costs 10-20 us, more than a small kernel runs)."""
    import torch
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(warm):
            fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(iters):
            fn()
    g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    g.replay()
    b.record()
    torch.cuda.synchronize()
    t = a.elapsed_time(b) / iters * 1e-3
    del g
    return t


def _lib_consts():
    from nvfp4_training_b200 import _lib
    return _lib


def isolated_kernels(cfg, T, peaks):
    """Time the GEMM and the quantizers alone (CUDA events on the launch stream), rotating operand
    sets so consecutive launches do not find their inputs in L2.  Returns the roofline object for
    the GEMM and a detail dict."""
    import torch
    from nvfp4_training_b200 import nvq
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(7)
    shapes = [(n, N, K) for n, N, K, _ in cfg.block_shapes()] + ([("head", cfg.vocab, cfg.d)] if cfg.lm_head else [])
    counts = {n: cfg.layers for n, _, _ in shapes}
    counts["head"] = 1
    detail, tot_flops, tot_time = {}, 0.0, 0.0

    def sets_for(nbytes):
        return max(2, min(8, int(256e6 // max(nbytes, 1)) + 1))

    # The quantizers are timed first, after a pause: they are issue-bound, so their rate follows the SM clock, and
    # right after seconds of back-to-back GEMMs the power controller still holds the clock down.  "Alone" here means
    # the kernel by itself on an otherwise idle GPU, like the burst figures of the measured peaks.
    torch.cuda.synchronize()
    time.sleep(1.5)
    # quantizers on the largest activation of a block: [T, 5632] X and [T, 11264] dY
    x = [torch.randn(T, 5632, generator=g, device=dev).bfloat16() for _ in range(4)]
    am = [nvq.amax(t) for t in x]
    n = T * 5632
    it = [0]

    def q(fn):
        def run():
            i = it[0] % 4
            it[0] += 1
            fn(x[i], am[i])
        return time_events(run, iters=20)
    t = q(lambda t, a: nvq.amax(t))
    detail["amax"] = {"elts": n, "us": t * 1e6, "gbs": n * 2.0 / t / 1e9}
    t = q(lambda t, a: nvq.quant_rows(t, am=a))
    detail["quant_rows_rn"] = {"elts": n, "us": t * 1e6, "gbs": n * 2.5625 / t / 1e9}
    HW = _lib_consts().ROUND_SR_HW          # the stack rounds gradients with the hardware convert
    t = q(lambda t, a: nvq.quant_rows(t, sr=True, seed=1, am=a, sr_mode=HW))
    detail["quant_rows_sr_hw"] = {"elts": n, "us": t * 1e6, "gbs": n * 2.5625 / t / 1e9}
    t = q(lambda t, a: nvq.quant_cols_rht(t, 0xA6B1, am=a))
    detail["quant_cols_rht_rn"] = {"elts": n, "us": t * 1e6, "gbs": n * 2.5625 / t / 1e9}
    t = q(lambda t, a: nvq.quant_cols_rht(t, 0xA6B1, sr=True, seed=1, am=a, sr_mode=HW))
    detail["quant_cols_rht_sr_hw"] = {"elts": n, "us": t * 1e6, "gbs": n * 2.5625 / t / 1e9}
    # the one-read tile quantizer (row + transposed operand): 2 B in, 2 x 0.5625 B out per element
    t = q(lambda t, a: nvq.quant_rows_cols_rht(t, 0xA6B1, am=a))
    detail["quant_tile_rn"] = {"elts": n, "us": t * 1e6, "gbs": n * 3.125 / t / 1e9}
    t = q(lambda t, a: nvq.quant_rows_cols_rht(t, 0xA6B1, sr=True, seed=1, seed_cols=2, am=a, sr_mode=HW))
    detail["quant_tile_sr_hw"] = {"elts": n, "us": t * 1e6, "gbs": n * 3.125 / t / 1e9}
    # row operand with per-row scales (the reference trainer's emitter): one read, no amax pass
    from nvfp4_training_b200 import emit
    rq = emit.RowQ(T, 5632)
    rng = torch.tensor([1, 0], dtype=torch.int32, device=dev)
    t = q(lambda t, a: emit.row_emit(t, rq, None))
    detail["emit_rows_rn"] = {"elts": n, "us": t * 1e6, "gbs": n * 2.5625 / t / 1e9}
    t = q(lambda t, a: emit.row_emit(t, rq, rng, sr=True))
    detail["emit_rows_sr"] = {"elts": n, "us": t * 1e6, "gbs": n * 2.5625 / t / 1e9}
    t = q(lambda t, a: emit.row_emit(t, rq, rng, sr="hw"))
    detail["emit_rows_sr_hw"] = {"elts": n, "us": t * 1e6, "gbs": n * 2.5625 / t / 1e9}
    # column operand with a delayed scale: RHT16 + quantization in one read, records the next amax
    cq = emit.ColQ(T, 5632)
    use = torch.full((1,), 16.0, dtype=torch.float32, device=dev)
    cur = torch.zeros(1, dtype=torch.int32, device=dev)
    t = q(lambda t, a: emit.col_emit(t, cq, use, cur, rng))
    detail["emit_cols_rn"] = {"elts": n, "us": t * 1e6, "gbs": n * 2.5625 / t / 1e9}
    t = q(lambda t, a: emit.col_emit(t, cq, use, cur, rng, sr=True))
    detail["emit_cols_sr"] = {"elts": n, "us": t * 1e6, "gbs": n * 2.5625 / t / 1e9}
    t = q(lambda t, a: emit.col_emit(t, cq, use, cur, rng, sr="hw"))
    detail["emit_cols_sr_hw"] = {"elts": n, "us": t * 1e6, "gbs": n * 2.5625 / t / 1e9}
    # producer-fused emitters of the reference's trainer.  swiglu_emit: [T, 2 x 5632] raw gate | up output (the
    # four [T, 5632] tensors above taken in pairs) -> row operand of silu(g) * u: 4 B in + 0.5625 B out per value
    gu = [torch.cat([x[0], x[1]], dim=1), torch.cat([x[2], x[3]], dim=1)]
    rs_in = torch.full((T,), 0.5, dtype=torch.float32, device=dev)
    one = torch.ones(1, dtype=torch.float32, device=dev)
    t = time_events(lambda: (it.__setitem__(0, it[0] + 1), emit.swiglu_emit(gu[it[0] % 2], rs_in, one, rq)), iters=20)
    detail["swiglu_emit"] = {"elts": n, "us": t * 1e6, "gbs": n * 4.5625 / t / 1e9}
    del gu
    # rms_emit: residual add + RMSNorm + row operand on [T, 2048]: x, y in, x_new out (2 B each), 0.5625 B of operand
    xs = [t_[:, :2048].contiguous() for t_ in x] + [t_[:, 2048:4096].contiguous() for t_ in x]
    xo = torch.empty(T, 2048, dtype=torch.bfloat16, device=dev)
    wn = torch.ones(2048, dtype=torch.bfloat16, device=dev)
    rq2 = emit.RowQ(T, 2048)
    n2 = T * 2048
    t = time_events(lambda: (it.__setitem__(0, it[0] + 1),
                             emit.rms_emit(xs[it[0] % 8], wn, rq2, y=xs[(it[0] + 3) % 8], ys=rs_in, ygw=one, xout=xo)), iters=24)
    detail["rms_emit_residual"] = {"elts": n2, "us": t * 1e6, "gbs": n2 * 6.5625 / t / 1e9}
    t = time_events(lambda: (it.__setitem__(0, it[0] + 1), emit.rms_emit(xs[it[0] % 8], wn, rq2)), iters=24)
    detail["rms_emit"] = {"elts": n2, "us": t * 1e6, "gbs": n2 * 2.5625 / t / 1e9}
    del xs, xo
    w = [torch.randn(11264, 2048, generator=g, device=dev).bfloat16() for _ in range(4)]
    it = [0]

    def wq():
        i = it[0] % 4
        it[0] += 1
        nvq.quant_w2d(w[i], am=am[0])
    t = time_events(wq, iters=20)
    detail["quant_w2d"] = {"elts": 11264 * 2048, "us": t * 1e6, "gbs": 11264 * 2048 * 3.125 / t / 1e9}
    for name, N, K in shapes:
        for pas, (M_, N_, K_, fp32) in {"fprop": (T, N, K, False), "dgrad": (T, K, N, False), "wgrad": (N, K, T, True)}.items():
            nset = sets_for((M_ + N_) * K_ * 0.5625 + M_ * N_ * (4 if fp32 else 2))
            ops = []
            for _ in range(nset):
                a = nvq.quant_rows(torch.randn(M_, K_, generator=g, device=dev).bfloat16())
                b = nvq.quant_rows(torch.randn(N_, K_, generator=g, device=dev).bfloat16())
                out = torch.zeros(M_, N_, dtype=torch.float32 if fp32 else torch.bfloat16, device=dev)
                ops.append((a, b, out))
            it = [0]

            def run():
                a, b, out = ops[it[0] % nset]
                it[0] += 1
                nvq.mm(a, b, out_dtype=out.dtype, out=out, accumulate=fp32)
            t = time_events(run, iters=max(10, 2 * nset))
            fl = 2.0 * M_ * N_ * K_
            detail[f"gemm_{name}_{pas}"] = {"M": M_, "N": N_, "K": K_, "us": t * 1e6, "tflops": fl / t / 1e12}
            if not fp32:
                # on-box comparator, a library call that is only timed: the reference's own GEMM
                # (torch._scaled_mm on the packed operands, llm-1b/nvq.py:92) on the same shape
                def run_lib():
                    a, b, _ = ops[it[0] % nset]
                    it[0] += 1
                    torch._scaled_mm(a.d, b.d.t(), a.s.view(-1), b.s.view(-1), out_dtype=torch.bfloat16)
                try:
                    tl = time_events(run_lib, iters=max(10, 2 * nset))
                    detail[f"gemm_{name}_{pas}"]["scaled_mm_tflops"] = fl / tl / 1e12
                except Exception as e:      # the comparator is optional: a torch build without FP4 _scaled_mm
                    detail[f"gemm_{name}_{pas}"]["scaled_mm_error"] = repr(e)[:120]
            tot_flops += fl * counts[name]
            tot_time += t * counts[name]
            del ops
    achieved = tot_flops / tot_time / 1e12
    fp4_peak = 4.0 * peaks["bf16_tflops"]
    roof = {"bound": "tensor", "achieved": achieved, "peak": fp4_peak, "unit": "TFLOP/s", "frac": achieved / fp4_peak,
            "traffic": None, "kernel": "gemm_nvf4_pair_kernel (tcgen05.mma cta_group::2 kind::mxf4nvf4 block16)",
            "peak_basis": "4 x cuBLAS bf16 burst TFLOP/s (dense FP4 : bf16 = 4 : 1 on B200)",
            "frac_of_nominal_9000": achieved / 9000.0,
            "how": "all 15 GEMM shapes of the step timed alone with CUDA events, weighted by launches per step",
            # `traffic` stays null: the figure is a launch mix, not one launch; DRAM bytes of single launches are in the
            # ncu summaries under profiles/ (gemm_*.md)
            "traffic_note": "launch mix: per-launch DRAM bytes are in profiles/gemm_*.md"}
    detail["hbm_peak_gbs"] = peaks["hbm_gbs"]
    return roof, detail


# ------------------------------------------------------------------------------------------ self-check
def _deq_rows(q, rows):
    """float64 [len(rows), C] block-scaled values (without the tensor scale) of rows of a packed operand, decoded
    with the package's pure-torch decoders (the reference's own test decoders, llm-1b/nvq.py:99-117)."""
    import torch
    from nvfp4_training_b200 import nvq
    R, C = q.d.shape[0], q.d.shape[1] * 2
    d = q.d.view(torch.uint8)[rows]
    sc = nvq.unswizzle(q.s, R, C // 16)[rows].contiguous().view(torch.float8_e4m3fn).double()
    tab = nvq._E2M1.to(device=d.device, dtype=torch.float64)
    v = torch.stack([tab[(d & 15).long()], tab[(d >> 4).long()]], -1).reshape(d.shape[0], C)
    return v * sc.repeat_interleave(16, 1)


def _gemm_rows_err(c, qa, qb, rows):
    """max over the sampled rows of |C - Y| / (tol_rel |Y| + 1e-6 max|Y|) and the relative Frobenius error, Y = FP64
    product of the dequantized operand bytes.  tol_rel = 1e-4 (FP32 out) or 2^-8 (bf16 out): <= 1 passes."""
    import torch
    all_rows = torch.arange(qb.d.shape[0], device=c.device)
    y = _deq_rows(qa, rows) @ _deq_rows(qb, all_rows).t() * (qa.gs.double() * qb.gs.double())
    got = c[rows].double()
    rel = 1e-4 if c.dtype == torch.float32 else 1.05 * 2.0 ** -8     # bf16: half an ulp is 2^-8 |y| at most
    worst = ((got - y).abs() / (rel * y.abs() + 1e-6 * y.abs().max())).max().item()
    fro = ((got - y).norm() / y.norm()).item()
    return worst, fro


def verify_step(stack, n_micro, world, rank):
    """Checks of the timed workload's results, after the timed region:
      kernels   y / dX / dW of one projection (down, 5632 -> 2048) at the step's own shapes, on 256 sampled rows each,
                against the FP64 product of their own dequantized operands (tolerances of the GPU tests);
      stack     the weight gradient the graph-replayed step leaves for that projection is bit-equal to an eager
                recomputation with the same device seeds (first microbatch stores, later ones add once);
      allreduce (N > 1) a slice of the all-reduced dW equals the sum of the ranks' local slices.
    Returns a dict with `ok`."""
    import torch
    import torch.distributed as dist
    from nvfp4_training_b200 import _lib, nvq
    from nvfp4_training_b200.linear import _RHT_SIGNS, linear_bwd, linear_fwd
    dev = stack.device
    out = {}
    p = stack.blocks[0][3]
    x, gy = stack.x_pool[p.name], stack.gy_pool[p.name]
    T = x.shape[0]
    g = torch.Generator(device=dev).manual_seed(5)
    rows_t = torch.sort(torch.randperm(T, generator=g, device=dev)[:256]).values
    rows_n = torch.sort(torch.randperm(p.N, generator=g, device=dev)[:256]).values
    am, ag = nvq.amax(x), nvq.amax(gy)
    qx, qxt = nvq.quant_rows_cols_rht(x, _RHT_SIGNS, am=am)
    qg, qgt = nvq.quant_rows_cols_rht(gy, _RHT_SIGNS, sr=True, seed=11, seed_cols=12, am=ag, sr_mode=stack.sr_mode)
    errs = {"y": _gemm_rows_err(nvq.mm(qx, p.q), qx, p.q, rows_t),
            "dx": _gemm_rows_err(nvq.mm(qg, p.qt), qg, p.qt, rows_t),
            "dw": _gemm_rows_err(nvq.mm(qgt, qxt, out_dtype=torch.float32), qgt, qxt, rows_n)}
    out["kernels"] = {k: {"worst_over_bound": v[0], "rel_fro": v[1]} for k, v in errs.items()}
    ok = all(v[0] <= 1.0 for v in errs.values())
    del qx, qxt, qg, qgt

    # stack result against an eager recomputation with the same seeds
    mc = stack.micro_count
    stack.step(n_micro, do_allreduce=False)
    local = p.gw.clone()
    def ends(t):          # the first and the last 65536 values: rows the first and the last rank own
        return torch.cat([t.view(-1)[:65536], t.view(-1)[-65536:]])
    local_head = ends(stack.blocks[-1][0].gw).clone()
    stack.micro_count = mc
    gw = torch.empty_like(p.gw)
    for m in range(n_micro):
        stack._bump_seeds()
        sd = stack.seeds[p.lid]
        _, am_x, qxt = linear_fwd(x, p.q, keep_xt=True, signs=_RHT_SIGNS)
        linear_bwd(None, am_x, gy, p.qt, sd[0:1], sd[1:2], gw_out=gw, signs=_RHT_SIGNS, sr_mode=stack.sr_mode,
                   overwrite=(m == 0), qxt=qxt)
    out["stack_equals_eager"] = bool(torch.equal(gw, local))
    ok = ok and out["stack_equals_eager"]

    if world > 1:
        stack.micro_count = mc
        stack.step(n_micro, do_allreduce=True)
        torch.cuda.synchronize()
        mine = torch.stack([ends(local), local_head])
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        want = torch.stack(gathered).double().sum(0)
        got = torch.stack([ends(p.gw), ends(stack.blocks[-1][0].gw)]).double()
        err = ((got - want).abs().max() / want.abs().max()).item()
        out["allreduce_max_err_over_max"] = err
        ok = ok and err <= 1e-6
    torch.cuda.synchronize()
    _lib.check_status()
    flag = torch.tensor([1.0 if ok else 0.0], device=dev)
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    out["ok"] = bool(flag.item() == 1.0)
    return out


def comm_breakdown(stack, n_micro, steps):
    """Where the time of a data-parallel step goes: the step with the all-reduce switched off, and the block-by-block
    all-reduces of all gradient buffers timed alone (CUDA events, this rank; the caller takes the max over ranks)."""
    import torch
    from nvfp4_training_b200.stack import allreduce_sum_

    def timed(fn, n):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.distributed.barrier()
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n
    stack.step(n_micro, False)
    ms_noar = timed(lambda: stack.step(n_micro, False), steps)

    def only_ar():
        for flat in reversed(stack.gw_flat):
            allreduce_sum_([flat], stack.group)
    only_ar()
    ms_ar = timed(only_ar, max(2, steps // 2))
    nbytes = sum(f.numel() * 4 for f in stack.gw_flat)
    return ms_noar, ms_ar, nbytes


# ------------------------------------------------------------------------------------------ configuration sweeps
def config_sweeps(cfg, peaks):
    """The other benchmark configurations, each timed with CUDA events on one GPU around a CUDA-graph replay of the
    launches (no host launch overhead in the figures; rotating operand sets larger than L2 where one set would fit):
      config2   every projection of one block at T = 4096: the whole layer (quantizers + 3 GEMMs, weights cached) and
                its three GEMMs alone
      config3   wgrad stress: dY [16384, 5632] stochastic + X [16384, 2048] nearest, RHT16 on both, FP32 dW
      config5   GEMM M = N = K in {4096, 8192, 16384}, M = 4096 with N, K in {2048, 5632, 49152} (with the library FP4
                GEMM behind torch._scaled_mm beside it); quantizers on 16 Mi .. 1 Gi elements, 1x16 / 16x16 / +RHT16 /
                +stochastic rounding and the one-read kernel that emits both operands
    """
    import torch
    from nvfp4_training_b200 import _lib, nvq
    from nvfp4_training_b200.linear import _RHT_SIGNS, linear_bwd, linear_fwd
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(11)
    HW = _lib.ROUND_SR_HW
    fp4_peak = 4.0 * peaks["bf16_tflops"]
    res = {"config2": {}, "config3": {}, "config5_gemm": {}, "config5_quant": {}}

    def rnd(r, c, scale=1.0):
        t = torch.randn(r, c, generator=g, device=dev, dtype=torch.bfloat16)
        return t if scale == 1.0 else (t.float() * scale).bfloat16()

    def gemm_time(M, N, K, fp32=False, lib=False):
        nset = max(2, min(6, int(300e6 // ((M + N) * K * 0.5625 + M * N * (4 if fp32 else 2))) + 1))
        ops = []
        for _ in range(nset):
            ops.append((nvq.quant_rows(rnd(M, K)), nvq.quant_rows(rnd(N, K)),
                        torch.empty(M, N, dtype=torch.float32 if fp32 else torch.bfloat16, device=dev)))
        it = [0]

        def run():
            a, b, o = ops[it[0] % nset]
            it[0] += 1
            nvq.mm(a, b, out_dtype=o.dtype, out=o)

        def run_lib():
            a, b, _ = ops[it[0] % nset]
            it[0] += 1
            torch._scaled_mm(a.d, b.d.t(), a.s.view(-1), b.s.view(-1), out_dtype=torch.bfloat16)
        t = time_graph(run, iters=max(8, 2 * nset))
        out = {"M": M, "N": N, "K": K, "us": t * 1e6, "tflops": 2.0 * M * N * K / t / 1e12,
               "frac_of_4x_bf16": 2.0 * M * N * K / t / 1e12 / fp4_peak}
        if lib and not fp32:
            try:
                tl = time_graph(run_lib, iters=max(8, 2 * nset))
                out["scaled_mm_tflops"] = 2.0 * M * N * K / tl / 1e12
            except Exception as e:
                out["scaled_mm_error"] = repr(e)[:100]
        return out

    torch.cuda.synchronize()
    time.sleep(1.5)      # the issue-bound quantizers are timed on an idle GPU, before the GEMM sweeps heat it
    # ---- config 5: quantizers
    hbm = peaks["hbm_gbs"]
    for label, R in (("16Mi", 2048), ("64Mi", 8192), ("256Mi", 32768), ("1Gi", 131072)):
        C = 8192
        n = R * C
        nset = max(1, min(8, int(300e6 // (n * 2)) + 1))
        xs = [rnd(R, C) for _ in range(nset)]
        am = nvq.amax(xs[0])
        it = [0]

        def t_of(fn, bpe):
            def run():
                it[0] += 1
                fn(xs[it[0] % nset])
            t = time_graph(run, iters=max(6, 2 * nset))
            return {"us": t * 1e6, "gbs": n * bpe / t / 1e9, "frac_hbm": n * bpe / t / 1e9 / hbm}
        res["config5_quant"][label] = {
            "elements": n,
            "amax": t_of(lambda t: nvq.amax(t), 2.0),
            "rows_1x16_rn": t_of(lambda t: nvq.quant_rows(t, am=am), 2.5625),
            "rows_1x16_sr": t_of(lambda t: nvq.quant_rows(t, sr=True, seed=1, am=am, sr_mode=HW), 2.5625),
            "cols_rht16_rn": t_of(lambda t: nvq.quant_cols_rht(t, _RHT_SIGNS, am=am), 2.5625),
            "cols_rht16_sr": t_of(lambda t: nvq.quant_cols_rht(t, _RHT_SIGNS, sr=True, seed=1, am=am, sr_mode=HW), 2.5625),
            "both_operands_rn": t_of(lambda t: nvq.quant_rows_cols_rht(t, _RHT_SIGNS, am=am), 3.125),
            "both_operands_sr": t_of(lambda t: nvq.quant_rows_cols_rht(t, _RHT_SIGNS, sr=True, seed=1, seed_cols=2, am=am, sr_mode=HW), 3.125),
            "w2d_16x16": t_of(lambda t: nvq.quant_w2d(t, am=am), 3.125),
        }
        del xs
        torch.cuda.empty_cache()
    # ---- config 2
    T = 4096
    projs = [("qkv", 3072, 2048), ("o_3072_to_2048", 2048, 3072), ("o_2048_to_2048", 2048, 2048),
             ("gate_up", 11264, 2048), ("down", 2048, 5632)]
    for name, N, K in projs:
        nset = 4
        xs = [rnd(T, K) for _ in range(nset)]
        gys = [rnd(T, N, 1e-3) for _ in range(nset)]
        q, qt = nvq.quant_w2d(rnd(N, K, 0.02))
        gw = torch.zeros(N, K, device=dev)
        it = [0]

        def layer():
            i = it[0] % nset
            it[0] += 1
            _, am, qxt = linear_fwd(xs[i], q, keep_xt=True)
            linear_bwd(None, am, gys[i], qt, 1, 2, gw_out=gw, sr_mode=HW, overwrite=True, qxt=qxt)
        t = time_graph(layer, iters=12)
        fl = 6.0 * T * N * K
        res["config2"][name] = {"T": T, "N": N, "K": K, "layer_us": t * 1e6, "layer_tflops": fl / t / 1e12,
                                "layer_frac_of_4x_bf16": fl / t / 1e12 / fp4_peak,
                                "fprop": gemm_time(T, N, K, lib=True), "dgrad": gemm_time(T, K, N, lib=True),
                                "wgrad": gemm_time(N, K, T, fp32=True)}
        del xs, gys
    # ---- config 3
    T, N, K = 16384, 5632, 2048
    gy, x = rnd(T, N, 1e-3), rnd(T, K)
    dw = torch.empty(N, K, device=dev)
    am_g, am_x = nvq.amax(gy), nvq.amax(x)

    def wgrad():
        qgt = nvq.quant_cols_rht(gy, _RHT_SIGNS, sr=True, seed=3, am=am_g, sr_mode=HW)
        qxt = nvq.quant_cols_rht(x, _RHT_SIGNS, am=am_x)
        nvq.mm(qgt, qxt, out_dtype=torch.float32, out=dw)
    t = time_graph(wgrad, iters=12)
    res["config3"] = {"T": T, "N": N, "K": K, "quant_plus_gemm_us": t * 1e6, "tflops": 2.0 * T * N * K / t / 1e12,
                      "gemm_alone": gemm_time(N, K, T, fp32=True)}
    exact = gy.double().t() @ x.double()
    res["config3"]["rel_err_vs_exact"] = ((dw.double() - exact).norm() / exact.norm()).item()
    del gy, x, dw, exact
    # ---- config 5: GEMM
    for n in (4096, 8192, 16384):
        res["config5_gemm"][f"square_{n}"] = gemm_time(n, n, n, lib=True)
    for N in (2048, 5632, 49152):
        for K in (2048, 5632, 49152):
            res["config5_gemm"][f"M4096_N{N}_K{K}"] = gemm_time(4096, N, K, lib=True)
    _lib.check_status()
    return res


def run_ours(args):
    import torch
    import torch.distributed as dist
    from nvfp4_training_b200 import _lib
    from nvfp4_training_b200.stack import LinearStack, StackConfig, shard_plan

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE {world}: launch with torch.distributed.run"
    torch.cuda.set_device(local)
    _lib.load().nvfp4_set_pdl(1 if args.pdl else 0)
    if args.comm_sms is None:
        # SMs kept out of the persistent backward grids (GEMM, quantizer) for NCCL.  The GEMM draws its tiles at run
        # time, so a grid that finds SMs taken by the collective needs no budget: the clusters that run share the work
        # and the late ones find none.  With 2 ranks the collective is in flight for about a third of the backward pass
        # and no budget wins (75.2-77.1 ms per step against 77.2-79.7 with 16 SMs set aside, same boxes); with 4 ranks
        # it is in flight half the time and a budget wins again (42.4 ms with 24 SMs, 42.7 with 32, 44.1 without: the
        # quantizer's CTAs own fixed shares of tiles and suffer from starting late); with 8 ranks it is in flight
        # almost all the time: 32 SMs (27.98 ms; 27.85 with 24, 28.28 with none, 30.81 with 16 SMs and 16 CTAs).
        args.comm_sms = 0 if world <= 2 else 24 if world < 8 else 32
    if not args.nccl_ctas:
        args.nccl_ctas = args.comm_sms if args.comm_sms > 0 else 32      # NCCL stays inside the SMs set aside for it
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_MAX_CTAS", str(args.nccl_ctas))
        # the collective's kernels go to a high-priority stream: when SMs come free between two kernels of the backward
        # pass, the collective's CTAs are placed first, so an exchange starts as soon as its block is done
        opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=not args.nccl_normal_priority)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), pg_options=opts)
    peaks, peak_src = load_peaks()

    cfg = StackConfig(layers=args.layers) if args.layers else StackConfig()
    plan = shard_plan(world, rank, GLOBAL_TOKENS, args.microbatch)
    mb, n_micro = plan["microbatch"], plan["n_micro"]
    stack = LinearStack(cfg, mb, torch.device("cuda", local), seed=0, input_seed=1000 + rank, use_graphs=not args.no_graphs,
                        comm_sms=args.comm_sms if world > 1 else 0, ar_blocks=args.ar_blocks,
                        wgrad_side_stream=not args.no_wgrad_stream, overlap_refresh=not args.no_overlap_refresh,
                        peer_reduce=args.peer_reduce and world > 1)
    if not args.no_graphs:
        stack.capture()
    do_ar = world > 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        stack.step(n_micro, do_ar)
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        stack.step(n_micro, do_ar)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if sampler else None
    _lib.check_status()

    # ---- end to end: the batch comes from pinned host memory every microbatch, a result goes back every step
    host_x = torch.randn(mb, cfg.d).bfloat16().pin_memory()
    host_out = torch.empty(1024, dtype=torch.float32).pin_memory()
    last = stack.blocks[-1][-1]
    launches_per_step = n_micro * stack.kernels_per_microbatch() + stack.n_proj * 2

    def e2e_step():
        stack.step(n_micro, do_ar, before_microbatch=lambda m: stack.x_pool["qkv"].copy_(host_x, non_blocking=True))
        host_out.copy_(last.gw.view(-1)[:1024], non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e2e_steps = max(1, min(args.steps, 5))
    e2e_step()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1) / e2e_steps

    # ---- where a data-parallel step's time goes (N > 1), and the self-check of the results
    ms_noar = ms_ar = 0.0
    ar_bytes = 0
    if world > 1 and (args.comm_breakdown or not args.skip_isolated):
        ms_noar, ms_ar, ar_bytes = comm_breakdown(stack, n_micro, max(2, min(args.steps, 5)))
    verify = None if args.no_verify else verify_step(stack, n_micro, world, rank)

    t = torch.tensor([ms, ms_e2e, ms_noar, ms_ar], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e, ms_noar, ms_ar = t.tolist()
    comm = None
    if world > 1 and ms_ar > 0:
        comm = {"step_without_allreduce_ms": ms_noar, "comm_exposed_ms": ms - ms_noar, "allreduce_alone_ms": ms_ar,
                "allreduce_bytes": ar_bytes, "gemm_sm_budget": args.comm_sms, "nccl_max_ctas": args.nccl_ctas,
                "reduce": ("weight-gradient GEMM epilogues add into the owner rank's row slab through peer memory; "
                           "NCCL barrier + in-place all-gather per block") if args.peer_reduce else "NCCL all-reduce per block",
                "allreduce_alone_busbw_gbs": 2.0 * (world - 1) / world * ar_bytes / (ms_ar * 1e-3) / 1e9,
                "how": "same step with the collective switched off; the block-by-block all-reduces of all gradient "
                       "buffers alone; CUDA events, max over ranks"}

    roof = detail = cpu = sweeps = mb4096 = emitter = None
    del stack
    torch.cuda.empty_cache()
    if world == 1 and not args.skip_isolated and mb != 4096:
        # the same step in 4096-row microbatches (the reference's microbatch size): 16x the launches
        plan2 = shard_plan(world, rank, GLOBAL_TOKENS, 4096)
        st2 = LinearStack(cfg, plan2["microbatch"], torch.device("cuda", local), seed=0, input_seed=1000 + rank,
                          use_graphs=not args.no_graphs)
        if not args.no_graphs:
            st2.capture()
        for _ in range(2):
            st2.step(plan2["n_micro"], False)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(3):
            st2.step(plan2["n_micro"], False)
        e1.record()
        torch.cuda.synchronize()
        ms2 = e0.elapsed_time(e1) / 3
        mb4096 = {"microbatch_tokens": 4096, "microbatches_per_rank": plan2["n_micro"], "ms_per_step": ms2,
                  "tokens_per_s": GLOBAL_TOKENS / (ms2 * 1e-3)}
        del st2
        torch.cuda.empty_cache()
        # the same step through the operand emitters of the reference's trainer (llm-1b/model2.py:430-480): row
        # operands with exact per-row scales, column operands with delayed per-tensor scales, no amax pass,
        # rs[row] * gs in the GEMM epilogue.  A second, separately labelled number: a different scaling contract.
        st3 = LinearStack(cfg, mb, torch.device("cuda", local), seed=0, input_seed=1000 + rank,
                          use_graphs=not args.no_graphs, mode="emit")
        if not args.no_graphs:
            st3.capture()
        for _ in range(2):
            st3.step(n_micro, False)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(3):
            st3.step(n_micro, False)
        e1.record()
        torch.cuda.synchronize()
        ms3 = e0.elapsed_time(e1) / 3
        _lib.check_status()
        emitter = {"contract": "per-row scales (row operands) + delayed per-tensor scales (column operands), no amax pass",
                   "microbatch_tokens": mb, "ms_per_step": ms3, "tokens_per_s": GLOBAL_TOKENS / (ms3 * 1e-3)}
        del st3
        torch.cuda.empty_cache()
    if rank == 0:
        if not args.skip_isolated:
            roof, detail = isolated_kernels(cfg, mb, peaks)
            roof["peak_source"] = peak_src
            if world == 1:
                sweeps = config_sweeps(cfg, peaks)
        if world == 1 and not args.no_cpu:
            threads = os.cpu_count() or 1
            cpu_reference_sample(64, threads)
            t0 = time.perf_counter()
            t_w, t_tok = cpu_reference_sample(256, threads)
            cpu = {"value": cpu_tokens_per_s(t_w, t_tok, 256), "unit": "tokens/s", "cores": threads, "kind": "port",
                   "sample": "one block's weight quant + 256 tokens fwd+bwd with the torch restatement of "
                             "small-model/model_ref.py, extrapolated by parameter count to the full step",
                   "sample_seconds": time.perf_counter() - t0}
    if world > 1:
        dist.barrier()
    if rank == 0:
        val = GLOBAL_TOKENS / (ms * 1e-3)
        flops = cfg.flops_per_token() * GLOBAL_TOKENS
        line = {
            "metric": "tokens/s", "value": val, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp4 (e2m1, ue4m3 block scales, fp32 accumulate)", "data": "synthetic",
            "config": workload_config(world, mb, n_micro),
            "tflops_per_gpu": flops / (ms * 1e-3) / world / 1e12,
            "frac_fp4_peak_per_gpu": flops / (ms * 1e-3) / world / 1e12 / (4.0 * peaks["bf16_tflops_sustained"]),
            "frac_fp4_nominal_9000": flops / (ms * 1e-3) / world / 1e12 / 9000.0,
            "e2e": {"value": GLOBAL_TOKENS / (ms_e2e * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": n_micro * mb * cfg.d * 2, "d2h_bytes_per_step": 4096, "steps": e2e_steps},
            # this library's kernels in the timed region: per microbatch and projection amax + tile quantizer +
            # GEMM (forward) and amax + tile quantizer + 2 GEMMs (backward); per step and weight amax + quant_w2d
            "gpu_launches": args.steps * launches_per_step,
            "clocks": clocks, "roofline": roof, "cpu_baseline": cpu, "verify": verify, "comm": comm,
            "step_with_4096_row_microbatches": mb4096, "step_through_operand_emitters": emitter, "detail": detail,
            "configs": sweeps,
        }
        print(json.dumps(line))
        if verify is not None and not verify["ok"]:
            sys.stderr.write("bench.py: result verification FAILED: " + json.dumps(verify) + "\n")
            sys.exit(3)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------ single-kernel cases
def run_case(args):
    """`--case gemm|quant|block`: a small, self-contained invocation of single kernels, meant for
    profiler captures (operands of a few hundred MB at most, each kernel launched `--iters` times, so
    a capture ends by itself).  Prints CUDA-event timings as one JSON line; not a benchmark number."""
    import torch
    from nvfp4_training_b200 import _lib, nvq
    from nvfp4_training_b200.linear import _RHT_SIGNS, linear_bwd, linear_fwd

    def timed(fn, iters):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / iters * 1e3

    a = args
    _lib.load().nvfp4_gemm_force_tile_n(a.tile)
    g = torch.Generator(device="cuda").manual_seed(0)
    out = {"case": a.case, "M": a.M, "N": a.N, "K": a.K}
    if a.case == "gemm":
        qa = nvq.quant_rows(torch.randn(a.M, a.K, generator=g, device="cuda").bfloat16())
        qb = nvq.quant_rows(torch.randn(a.N, a.K, generator=g, device="cuda").bfloat16())
        dt = torch.float32 if a.fp32 else torch.bfloat16
        c = torch.empty(a.M, a.N, dtype=dt, device="cuda")
        us = timed(lambda: nvq.mm(qa, qb, out_dtype=dt, out=c), a.iters)
        out.update(us=us, tflops=2.0 * a.M * a.N * a.K / us / 1e6)
    elif a.case == "quant":
        # `--sets` input tensors [M, N] taken in turn: with sets * M * N * 2 bytes well above the L2 size
        # every launch reads its input from HBM
        xs = [torch.randn(a.M, a.N, generator=g, device="cuda").bfloat16() for _ in range(a.sets)]
        turn = [0]

        def nxt():
            turn[0] += 1
            return xs[turn[0] % a.sets]
        am = nvq.amax(xs[0])
        n = a.M * a.N
        HW, S = _lib.ROUND_SR_HW, _RHT_SIGNS
        cases = (
            ("amax", lambda x: nvq.amax(x), 2.0),
            ("quant_rows_rn", lambda x: nvq.quant_rows(x, am=am), 2.5625),
            ("quant_rows_sr_hw", lambda x: nvq.quant_rows(x, sr=True, seed=1, am=am, sr_mode=HW), 2.5625),
            ("tile_rows+cols_sr_hw", lambda x: nvq.quant_rows_cols_rht(x, S, sr=True, seed=1, seed_cols=2, am=am, sr_mode=HW), 3.125),
            ("tile_cols_sr_hw", lambda x: nvq.quant_rows_cols_rht(x, S, sr=True, seed=1, seed_cols=2, am=am, sr_mode=HW, want=(False, True)), 2.5625),
            ("tile_rows_sr_hw", lambda x: nvq.quant_rows_cols_rht(x, S, sr=True, seed=1, seed_cols=2, am=am, sr_mode=HW, want=(True, False)), 2.5625),
            ("tile_rows+cols_rn", lambda x: nvq.quant_rows_cols_rht(x, S, am=am), 3.125),
            ("tile_cols_rn", lambda x: nvq.quant_rows_cols_rht(x, S, am=am, want=(False, True)), 2.5625),
            ("tile_rows_rn", lambda x: nvq.quant_rows_cols_rht(x, S, am=am, want=(True, False)), 2.5625),
        )
        if a.N % 256 == 0:
            from nvfp4_training_b200 import emit
            rq = emit.RowQ(a.M, a.N)
            rng = torch.tensor([1, 0], dtype=torch.int32, device="cuda")
            cases = cases + (("emit_rows_rn", lambda x: emit.row_emit(x, rq, None), 2.5625),
                             ("emit_rows_sr", lambda x: emit.row_emit(x, rq, rng, sr=True), 2.5625),
                             ("emit_rows_hw", lambda x: emit.row_emit(x, rq, rng, sr="hw"), 2.5625))
            one = torch.ones(1, dtype=torch.float32, device="cuda")
            rs_in = torch.full((a.M,), 0.5, dtype=torch.float32, device="cuda")
            if a.N in (1024, 2048, 4096):
                wn = torch.ones(a.N, dtype=torch.bfloat16, device="cuda")
                xo = torch.empty(a.M, a.N, dtype=torch.bfloat16, device="cuda")
                cases = cases + (("rms_emit_operand", lambda x: emit.rms_emit(x, wn, rq), 2.5625),
                                 ("rms_emit_residual", lambda x: emit.rms_emit(x, wn, rq, y=xs[0], ys=rs_in, ygw=one, xout=xo), 6.5625))
            if a.only and "swiglu" in a.only:
                gus = [torch.cat([x_, x_], dim=1) for x_ in xs]          # raw gate | up output [M, 2N]
                cases = cases + (("swiglu_emit", lambda x: emit.swiglu_emit(gus[turn[0] % a.sets], rs_in, one, rq), 4.5625),)
            if a.M % 256 == 0:
                cq = emit.ColQ(a.M, a.N)
                use = torch.full((1,), 16.0, dtype=torch.float32, device="cuda")
                cur = torch.zeros(1, dtype=torch.int32, device="cuda")
                cases = cases + (("emit_cols_rn", lambda x: emit.col_emit(x, cq, use, cur, rng), 2.5625),
                                 ("emit_cols_sr", lambda x: emit.col_emit(x, cq, use, cur, rng, sr=True), 2.5625))
        for name, fn, bpe in cases:
            if a.only and a.only not in name:
                continue
            us = timed(lambda: fn(nxt()), a.iters)
            out[name] = {"us": us, "gbs": n * bpe / us / 1e3}
        if not a.only:
            w = torch.randn(a.N, a.K, generator=g, device="cuda").bfloat16()
            us = timed(lambda: nvq.quant_w2d(w), a.iters)
            out["amax+quant_w2d"] = {"us": us, "gbs": a.N * a.K * 5.125 / us / 1e3}
    else:
        x = torch.randn(a.M, a.K, generator=g, device="cuda").bfloat16()
        w = (torch.randn(a.N, a.K, generator=g, device="cuda") * 0.02).bfloat16()
        gy = (torch.randn(a.M, a.N, generator=g, device="cuda") * 1e-3).bfloat16()
        q, qt = nvq.quant_w2d(w)
        gw = torch.zeros(a.N, a.K, device="cuda")

        def step():
            _, am = linear_fwd(x, q)
            linear_bwd(x, am, gy, qt, 1, 2, gw_out=gw)
        us = timed(step, a.iters)
        out.update(us=us, tflops=6.0 * a.M * a.N * a.K / us / 1e6)
    _lib.check_status()
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--microbatch", type=int, default=65536,
                    help="rows per microbatch (default: the whole local batch; 148.0 ms per step at N = 1 against 150.8 with 32768 and 156.1 with 16384)")
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer blocks (not a valid bench number)")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--ar-blocks", type=int, default=1, help="transformer blocks per gradient all-reduce")
    ap.add_argument("--comm-sms", type=int, default=None,
                    help="SMs kept out of the persistent backward grids for NCCL when N > 1 (default: 0 at N = 2, 24 at N = 4, 32 at N >= 8)")
    ap.add_argument("--nccl-normal-priority", action="store_true", help="N > 1: NCCL's stream at normal instead of high priority")
    ap.add_argument("--comm-breakdown", action="store_true",
                    help="N > 1: time the step without the exchange and the exchange alone even with --skip-isolated")
    ap.add_argument("--peer-reduce", action="store_true",
                    help="N > 1: reduce-scatter inside the weight-gradient GEMM epilogues (adds into the owner rank's memory "
                         "over NVLink) + all-gather, instead of NCCL all-reduce")
    ap.add_argument("--no-overlap-refresh", action="store_true",
                    help="re-quantize all weights at the start of a step instead of block by block behind the backward pass")
    ap.add_argument("--nccl-ctas", type=int, default=0, help="NCCL_MAX_CTAS (default: --comm-sms, or 32 when no SMs are set aside)")
    ap.add_argument("--no-wgrad-stream", action="store_true",
                    help="weight-gradient GEMMs on the main stream instead of a side stream beside the dgrad chain")
    ap.add_argument("--pdl", action="store_true", help="programmatic dependent launch of the library's kernels (off by default)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--skip-isolated", action="store_true",
                    help="skip the isolated-kernel legs, the configuration sweeps and the communication breakdown (for profiler runs)")
    ap.add_argument("--no-verify", action="store_true", help="skip the self-check of the results after the timed region")
    ap.add_argument("--case", default=None, choices=["gemm", "quant", "block"],
                    help="run one small single-kernel case instead of the benchmark (for profiler captures)")
    ap.add_argument("--M", type=int, default=8192)
    ap.add_argument("--N", type=int, default=3072)
    ap.add_argument("--K", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--fp32", action="store_true", help="--case gemm: FP32 output")
    ap.add_argument("--tile", type=int, default=0, help="--case gemm: forced tile variant (nvfp4_gemm_force_tile_n)")
    ap.add_argument("--sets", type=int, default=1, help="--case quant: input tensors taken in turn")
    ap.add_argument("--only", default="", help="--case quant: run only the sub-cases whose name contains this")
    args = ap.parse_args()
    if args.case:
        run_case(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
