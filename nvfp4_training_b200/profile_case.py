"""Small, self-contained invocations of single kernels for profilers.

    python -m nvfp4_training_b200.profile_case --what gemm --M 8192 --N 3072 --K 2048 --iters 3
    python -m nvfp4_training_b200.profile_case --what quant --M 8192 --N 5632 --iters 3
    python -m nvfp4_training_b200.profile_case --what block --M 8192

Operands are a few hundred MB at most (larger than L2, far below device memory) and each kernel is
launched `iters` times, so a capture ends by itself.  Prints CUDA-event timings as one JSON line.
"""
import argparse
import json

import torch

from . import _lib, nvq
from .linear import _RHT_SIGNS, linear_bwd, linear_fwd


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="gemm", choices=["gemm", "quant", "block"])
    ap.add_argument("--M", type=int, default=8192)
    ap.add_argument("--N", type=int, default=3072)
    ap.add_argument("--K", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--fp32", action="store_true")
    ap.add_argument("--tile", type=int, default=0)
    ap.add_argument("--sets", type=int, default=1)
    a = ap.parse_args()
    _lib.load().nvfp4_gemm_force_tile_n(a.tile)
    g = torch.Generator(device="cuda").manual_seed(0)
    out = {"what": a.what, "M": a.M, "N": a.N, "K": a.K}
    if a.what == "gemm":
        qa = nvq.quant_rows(torch.randn(a.M, a.K, generator=g, device="cuda").bfloat16())
        qb = nvq.quant_rows(torch.randn(a.N, a.K, generator=g, device="cuda").bfloat16())
        dt = torch.float32 if a.fp32 else torch.bfloat16
        c = torch.empty(a.M, a.N, dtype=dt, device="cuda")
        us = timed(lambda: nvq.mm(qa, qb, out_dtype=dt, out=c), a.iters)
        out.update(us=us, tflops=2.0 * a.M * a.N * a.K / us / 1e6)
    elif a.what == "quant":
        # `--sets` input tensors taken in turn: with sets * M * N * 2 bytes well above the L2 size
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
            ("quant_rows_sr", lambda x: nvq.quant_rows(x, sr=True, seed=1, am=am), 2.5625),
            ("quant_cols_rht_rn", lambda x: nvq.quant_cols_rht(x, S, am=am), 2.5625),
            ("quant_cols_rht_sr", lambda x: nvq.quant_cols_rht(x, S, sr=True, seed=1, am=am), 2.5625),
            ("quant_rows_sr_hw", lambda x: nvq.quant_rows(x, sr=True, seed=1, am=am, sr_mode=HW), 2.5625),
            ("quant_cols_rht_sr_hw", lambda x: nvq.quant_cols_rht(x, S, sr=True, seed=1, am=am, sr_mode=HW), 2.5625),
            ("tile_rows+cols_sr_hw", lambda x: nvq.quant_rows_cols_rht(x, S, sr=True, seed=1, seed_cols=2, am=am, sr_mode=HW), 3.125),
            ("tile_cols_sr_hw", lambda x: nvq.quant_rows_cols_rht(x, S, sr=True, seed=1, seed_cols=2, am=am, sr_mode=HW, want=(False, True)), 2.5625),
            ("tile_rows_sr_hw", lambda x: nvq.quant_rows_cols_rht(x, S, sr=True, seed=1, seed_cols=2, am=am, sr_mode=HW, want=(True, False)), 2.5625),
            ("tile_rows+cols_rn", lambda x: nvq.quant_rows_cols_rht(x, S, am=am), 3.125),
            ("tile_cols_rn", lambda x: nvq.quant_rows_cols_rht(x, S, am=am, want=(False, True)), 2.5625),
        )
        if a.N % 256 == 0:
            from . import emit
            rq = emit.RowQ(a.M, a.N)
            rng = torch.tensor([1, 0], dtype=torch.int32, device="cuda")
            cases = cases + (("emit_rows_rn", lambda x: emit.row_emit(x, rq, None), 2.5625),
                             ("emit_rows_sr", lambda x: emit.row_emit(x, rq, rng, sr=True), 2.5625))
            if a.M % 256 == 0:
                cq = emit.ColQ(a.M, a.N)
                use = torch.full((1,), 16.0, dtype=torch.float32, device="cuda")
                cur = torch.zeros(1, dtype=torch.int32, device="cuda")
                cases = cases + (("emit_cols_rn", lambda x: emit.col_emit(x, cq, use, cur, rng), 2.5625),
                                 ("emit_cols_sr", lambda x: emit.col_emit(x, cq, use, cur, rng, sr=True), 2.5625))
        for name, fn, bpe in cases:
            us = timed(lambda: fn(nxt()), a.iters)
            out[name] = {"us": us, "gbs": n * bpe / us / 1e3}
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


if __name__ == "__main__":
    main()
