"""Host-side logic of the data-parallel path on CPU ranks (gloo, world size 2): row sharding and
the FP32 weight-gradient all-reduce.  With round-to-nearest and a shared tensor amax the sum of the
per-rank wgrads equals the single-rank wgrad over all rows up to FP32 summation order."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nvfp4_training_b200.stack import StackConfig, allreduce_sum_, shard_plan
from oracle import torch_ref as T


def test_shard_plan():
    p = [shard_plan(4, r, 65536, 8192) for r in range(4)]
    assert [q["row0"] for q in p] == [0, 16384, 32768, 49152]
    assert all(q["rows"] == 16384 and q["microbatch"] == 8192 and q["n_micro"] == 2 for q in p)
    assert shard_plan(8, 7, 65536, 16384)["microbatch"] == 8192
    with pytest.raises(ValueError):
        shard_plan(3, 0, 65536, 8192)
    with pytest.raises(ValueError):
        shard_plan(2, 0, 65536, 5000)


def test_stack_config_counts():
    c = StackConfig()
    assert c.n_params() == 1002438656 and abs(c.flops_per_token() / 1e9 - 6.0146) < 1e-3
    assert [(n, k) for _, n, k, _ in c.block_shapes()] == [(3072, 2048), (2048, 2048), (11264, 2048), (2048, 5632)]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    g = torch.Generator().manual_seed(0)
    rows, N, K = 512, 128, 128
    x = torch.randn(rows, K, generator=g).bfloat16()
    gy = (torch.randn(rows, N, generator=g) * 1e-3).bfloat16()
    plan = shard_plan(world, rank, rows, 128, seq_len=256)
    sl = slice(plan["row0"], plan["row0"] + plan["rows"])
    ax, ag = x.float().abs().max() * 4, gy.float().abs().max() * 4          # shared amax -> same scales
    gw = torch.zeros(N, K)
    for m in range(plan["n_micro"]):
        r = slice(sl.start + m * plan["microbatch"], sl.start + (m + 1) * plan["microbatch"])
        gt = T.nvfp4_1d(T.rht16_t(gy[r], 0xA5C3), gamax=ag)
        xt = T.nvfp4_1d(T.rht16_t(x[r], 0xA5C3), gamax=ax)
        gw += gt @ xt.t()
    allreduce_sum_([gw])
    if rank == 0:
        full = T.nvfp4_1d(T.rht16_t(gy, 0xA5C3), gamax=ag) @ T.nvfp4_1d(T.rht16_t(x, 0xA5C3), gamax=ax).t()
        out.put((float((gw - full).norm() / full.norm()), plan))
    dist.destroy_process_group()


def test_sharded_wgrad_allreduce_matches_single_rank():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    err, plan = out.get()
    assert plan["n_micro"] == 2 and err < 1e-6
