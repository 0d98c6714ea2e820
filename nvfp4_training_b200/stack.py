"""The NVFP4 linear layers of the 1B architecture as one data-parallel workload.

Shapes follow the reference model (llm-1b/model.py:18-32 `Config`, :135-149 `Block`): per block
qkv 2048->3072, o 2048->2048, gate/up 2048->11264, down 5632->2048, 20 blocks, plus the LM head
2048->49152 run as an NVFP4 linear.  Everything between the linears (norms, attention, SwiGLU,
loss) is outside this path: each projection reads its input and output-gradient from seeded
synthetic pools of the right shape and distribution.

One process per GPU.  Tokens are sharded by rows, weights replicated; fprop and dgrad need no
communication.  The FP32 weight gradients are accumulated in place over the rank's microbatches and
all-reduced (sum) once per step, block by block on a side stream as soon as the block's last
backward has been enqueued, so NCCL overlaps the remaining backward GEMMs.

Launch overhead: each block's four forwards, and its four backwards, are captured once into CUDA
graphs that share one memory pool and are replayed per microbatch; stochastic-rounding seeds are
read from device memory so every replay rounds with fresh bits.
"""
from dataclasses import dataclass

import torch

from . import _lib, emit, nvq
from .linear import _RHT_SIGNS, linear_bwd, linear_fwd

EMIT_MARGIN = 2.0      # delayed column scales use the last observed amax times this (llm-1b/model2.py:13,497-499)


@dataclass
class StackConfig:
    vocab: int = 49152
    d: int = 2048
    layers: int = 20
    heads: int = 16
    kv_heads: int = 4
    ff: int = 5632
    lm_head: bool = True

    @property
    def hd(self):
        return self.d // self.heads

    def block_shapes(self):
        """(name, N out-features, K in-features, init std) of one block (llm-1b/model.py:139-149)."""
        std, out_std = 0.02, 0.02 / (2 * self.layers) ** 0.5
        return [("qkv", (self.heads + 2 * self.kv_heads) * self.hd, self.d, std),
                ("o", self.d, self.heads * self.hd, out_std),
                ("gu", 2 * self.ff, self.d, std),
                ("down", self.d, self.ff, out_std)]

    def flops_per_token(self):
        per_block = sum(6 * n * k for _, n, k, _ in self.block_shapes())
        return per_block * self.layers + (6 * self.vocab * self.d if self.lm_head else 0)

    def n_params(self):
        return sum(n * k for _, n, k, _ in self.block_shapes()) * self.layers + (self.vocab * self.d if self.lm_head else 0)


def shard_plan(world, rank, global_tokens, microbatch, seq_len=2048):
    """Row sharding of the global batch: whole sequences per rank, the rank's rows cut into equal
    microbatches.  RHT16 blocks (16 rows) and 128-row tiles never straddle ranks or microbatches."""
    n_seq = global_tokens // seq_len
    if global_tokens % seq_len or n_seq % world:
        raise ValueError(f"{global_tokens} tokens = {n_seq} sequences do not split over {world} ranks")
    t_local = global_tokens // world
    mb = min(microbatch, t_local)
    if mb % 128 or t_local % mb:
        raise ValueError(f"microbatch {mb} must be a multiple of 128 and divide the {t_local} local tokens")
    return {"row0": rank * t_local, "rows": t_local, "microbatch": mb, "n_micro": t_local // mb}


def allreduce_sum_(tensors, group=None):
    """In-place FP32 sum of the weight gradients over the data-parallel group: the one exchange of
    this path.  Works on any backend (NCCL on GPUs, gloo in the CPU tests)."""
    for t in tensors:
        assert t.dtype == torch.float32
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.SUM, group=group)
    return tensors


class _Proj:
    __slots__ = ("name", "N", "K", "w", "q", "qt", "gw", "lid", "am_x", "y", "gx", "qxt", "wq", "cx", "owners")


def student_t(shape, gen, device, df=3):
    z = torch.randn(shape, generator=gen, device=device)
    chi = torch.randn((df,) + tuple(shape), generator=gen, device=device).square_().sum(0)
    return z / torch.sqrt(chi / df)


class LinearStack:
    def __init__(self, cfg: StackConfig, microbatch: int, device, seed=0, use_graphs=True, group=None,
                 sr_mode=_lib.ROUND_SR_HW, comm_sms=0, ar_blocks=1, input_seed=None, mode="tensor", wgrad_side_stream=True, overlap_refresh=True,
                 peer_reduce=False):
        """`seed` initialises the weights (the same on every rank of a data-parallel job: replicated
        weights), `input_seed` the synthetic activation / gradient pools (different per rank: each rank
        holds its own rows of the batch; default seed + 1000).
        `mode`: "tensor" = the per-tensor-scale contract of llm-1b/model.py (amax pass + one-read quantizer);
        "emit" = the operand emitters of the reference's trainer (llm-1b/model2.py:430-480): row operands with exact
        per-row scales, column operands with delayed per-tensor scales, no amax pass, `rs[row] * gs` applied in the
        GEMM epilogue.
        `peer_reduce` (NCCL jobs on one NVLink domain): the reduce half of the gradient all-reduce moves into the
        weight-gradient GEMMs: every rank owns a row slab of each dW, the GEMM epilogues add their tiles straight into
        the owners' memory (symmetric memory, `nvfp4_gemm_scatter_rows`), and what is left for the collective library
        is one barrier and an in-place all-gather of the slabs per block."""
        assert mode in ("tensor", "emit")
        self.mode = mode
        self.peer_reduce = bool(peer_reduce)
        # a block's weights are re-quantized on the side stream right after the block's gradients are reduced (where
        # a trainer would apply the block's optimizer update first), under the rest of the backward pass, instead of
        # all weights at the start of the next step
        self.overlap_refresh = overlap_refresh
        self.after_reduce = None      # optional callable(block_index, projs), run on the side stream between a block's
        #                               all-reduce and its re-quantization: the place of the block's optimizer update
        self._weights_fresh = False
        self.graphs_refresh_blk = None
        # weight-gradient GEMMs run on a side stream, joined at the end of each block's backward: they are off the
        # critical chain amax -> quantize -> dgrad, and fill the SMs that chain's kernels leave idle in their last waves
        self.wgrad_stream = torch.cuda.Stream(device=device) if wgrad_side_stream else None
        # emitter mode rounds gradients with the hardware convert ("hw"); True selects the reference's dither sequences
        self.emit_sr = "hw" if sr_mode == _lib.ROUND_SR_HW else True
        self.comm_sms = comm_sms     # SMs left to NCCL while backward GEMMs and the all-reduce overlap
        self.ar_blocks = max(1, ar_blocks)   # transformer blocks per gradient all-reduce
        self.cfg, self.T, self.device, self.group = cfg, microbatch, torch.device(device), group
        self.sr_mode = sr_mode       # gradients: hardware cvt.rs stochastic rounding, counter-based random words
        self.use_graphs = use_graphs
        gen = torch.Generator(device=self.device).manual_seed(seed)
        self.blocks = []
        lid = 0
        names = cfg.block_shapes()
        for b in range(cfg.layers):
            projs = []
            for name, N, K, std in names:
                projs.append(self._make_proj(name, N, K, std, lid, gen))
                lid += 1
            self.blocks.append(projs)
        if cfg.lm_head:
            self.blocks.append([self._make_proj("head", cfg.vocab, cfg.d, 0.02, lid, gen)])
            lid += 1
        self.n_proj = lid
        self.w_am = torch.zeros(lid, dtype=torch.float32, device=self.device)           # amax of each weight
        self.am_words = torch.zeros(2, lid, dtype=torch.float32, device=self.device)   # amax of x / of dy per projection
        # the weight gradients of `ar_blocks` consecutive blocks live in one flat FP32 buffer, so that
        # their all-reduce is one collective (the LM head keeps a buffer of its own: it is first in
        # the backward order and its collective should start at once)
        self.gw_flat, self.ar_after = [], {}       # ar_after[block index] = flat buffer to reduce once that block is done
        nb = cfg.layers
        groups = [list(range(b, min(b + self.ar_blocks, nb))) for b in range(0, nb, self.ar_blocks)]
        if cfg.lm_head:
            groups.append([nb])
        arena, arena_off = None, 0
        if self.peer_reduce:
            arena = self._peer_arena(sum(p.N * p.K for projs in self.blocks for p in projs))
        for grp in groups:
            projs = [p for b in grp for p in self.blocks[b]]
            n_flat = sum(p.N * p.K for p in projs)
            if arena is None:
                flat = torch.zeros(n_flat, dtype=torch.float32, device=self.device)
            else:
                flat = arena[arena_off:arena_off + n_flat]
                self._peer_views(projs, arena_off)
                arena_off += n_flat
            off = 0
            for p in projs:
                p.gw = flat[off:off + p.N * p.K].view(p.N, p.K)
                off += p.N * p.K
            self.gw_flat.append(flat)
            self.ar_after[grp[0]] = flat           # backward walks the blocks downwards: the group's lowest block is last
        # synthetic pools: X ~ N(0,1) bf16, dY ~ Student-t(3) * 1e-3 bf16, one per projection kind
        gen_in = torch.Generator(device=self.device).manual_seed(seed + 1000 if input_seed is None else input_seed)
        self.x_pool, self.gy_pool = {}, {}
        for name, N, K, _ in names + ([("head", cfg.vocab, cfg.d, 0.02)] if cfg.lm_head else []):
            self.x_pool[name] = torch.randn(self.T, K, generator=gen_in, device=self.device).bfloat16()
            self.gy_pool[name] = (student_t((self.T, N), gen_in, self.device) * 1e-3).bfloat16()
        # per-projection SR seeds in device memory: [n_proj, 2] = (seed, seed ^ 0x5bd1e995) (llm-1b/model.py:59,66)
        self.seeds = torch.zeros(self.n_proj, 2, dtype=torch.int32, device=self.device)
        self._lids = torch.arange(self.n_proj, dtype=torch.int64, device=self.device) * 7919
        # emitter mode: delayed amax of the two column operands of every projection (x, gy), the observed
        # values of the running microbatch, and the device words the emitters read (seed, Hadamard signs)
        self.amax_use = torch.full((self.n_proj, 2), 1e9, dtype=torch.float32, device=self.device)
        self.amax_cur = torch.zeros(self.n_proj, 2, dtype=torch.int32, device=self.device)
        self.rng = torch.tensor([0, _RHT_SIGNS], dtype=torch.int32, device=self.device)
        self._calibrated = False
        self.micro_count = 0
        self._bump_seeds()
        self.comm_stream = torch.cuda.Stream(device=self.device)
        # a block's optimizer hook and weight re-quantization run on a stream of their own, behind the block's
        # collective: on the collective's stream they would sit between two blocks' exchanges and keep the links
        # idle meanwhile (with 8 ranks the exchanges fill most of the backward pass)
        self.refresh_stream = torch.cuda.Stream(device=self.device)
        self.graphs_fwd = self.graphs_bwd = self.graphs_bwd_scatter = None
        self.graph_refresh = None
        self.launches_per_micro = 0

    def _make_proj(self, name, N, K, std, lid, gen):
        p = _Proj()
        p.name, p.N, p.K, p.lid = name, N, K, lid
        w = torch.empty(N, K, device=self.device)
        torch.nn.init.trunc_normal_(w, std=std, a=-3 * std, b=3 * std, generator=gen)
        p.w = w.bfloat16()
        p.gw = None      # a view of the block's flat gradient buffer, set by the constructor
        p.q = p.qt = p.am_x = p.y = p.gx = p.qxt = p.wq = p.cx = p.owners = None
        return p

    # ------------------------------------------------------------------ gradients reduced through peer memory
    def _peer_arena(self, n_floats):
        """One FP32 buffer for all weight gradients, at the same offsets on every rank, mapped into every rank's
        address space."""
        import os
        import torch.distributed as dist
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")      # plain peer stores only: no multicast binding
        import torch.distributed._symmetric_memory as symm
        assert dist.is_initialized() and dist.get_backend(self.group) == "nccl" and self.ar_blocks == 1
        grp = self.group if self.group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(grp), dist.get_rank(grp)
        assert 1 <= self.world <= 8
        arena = symm.empty(n_floats, dtype=torch.float32, device=self.device)
        self._peer_handle = symm.rendezvous(arena, grp)
        self._peer_base = [int(self._peer_handle.buffer_ptrs[r]) for r in range(self.world)]
        assert self._peer_base[self.rank] == arena.data_ptr()
        arena.zero_()
        self._bar_word = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._peer_ready = None
        return arena

    def _peer_views(self, projs, first_float):
        off = first_float
        for p in projs:
            assert p.N % 256 == 0 and (p.N // self.world) % 128 == 0, (p.name, p.N, self.world)
            p.owners = [base + 4 * off for base in self._peer_base]
            off += p.N * p.K

    def _slab(self, p):
        n = p.N // self.world
        return p.gw[self.rank * n:(self.rank + 1) * n]

    def _peer_barrier(self):
        torch.distributed.all_reduce(self._bar_word, group=self.group)

    def _peer_begin_step(self):
        """On the side stream, beside the forward pass: once every rank is past the previous step, clear the slabs
        this rank owns, and let no rank start adding before all slabs are clear."""
        cur = torch.cuda.current_stream()
        self.comm_stream.wait_stream(cur)
        with torch.cuda.stream(self.comm_stream):
            self._peer_barrier()
            for projs in self.blocks:
                for p in projs:
                    self._slab(p).zero_()
            self._peer_barrier()
            self._peer_ready = torch.cuda.Event()
            self._peer_ready.record()

    def _peer_finish_block(self, projs):
        """On the side stream, behind the block's last weight-gradient GEMM of this rank: once every rank is there,
        all contributions have landed in the owners' slabs; the in-place all-gather hands every rank all slabs."""
        self._peer_barrier()
        for p in projs:
            torch.distributed.all_gather_into_tensor(p.gw.view(-1), self._slab(p).reshape(-1), group=self.group)

    # ------------------------------------------------------------------ per-step pieces
    def _bump_seeds(self):
        """seed = (LinCtx.seed * 1000003 + lid * 7919) & 0xFFFFFFFF, LinCtx.seed = microbatch counter."""
        s = (self._lids + self.micro_count * 1000003) & 0xFFFFFFFF
        both = torch.stack([s, s ^ 0x5BD1E995], 1)
        self.seeds.copy_(torch.where(both >= 2 ** 31, both - 2 ** 32, both).to(torch.int32))
        self.rng[0] = (self.micro_count * 1000003 + 12345) % (2 ** 31)
        self.micro_count += 1

    def roll_amax(self):
        """Delayed scaling: this microbatch's observed RHT-domain amax (x margin) scales the next one
        (llm-1b/model2.py:497-499)."""
        torch.mul(self.amax_cur.view(torch.float32).clamp(min=1e-30), EMIT_MARGIN, out=self.amax_use)
        self.amax_cur.zero_()

    def _refresh_block(self, projs):
        lo, hi = projs[0].lid, projs[-1].lid + 1
        self.w_am[lo:hi].zero_()            # one fill for the block's amax words: the rest is a chain of kernels
        for p in projs:
            am = nvq.amax(p.w, out=self.w_am[p.lid:p.lid + 1], clear=False)
            if p.q is None:
                p.q, p.qt = nvq.quant_w2d(p.w, am=am)
            else:
                nvq.quant_w2d(p.w, am=am, out=(p.q, p.qt))      # in place: captured graphs keep these buffers

    def refresh_weights(self):
        """Quantize every weight once per optimizer step (the small-model/fp4torch.py:71-84 scheme).
        After `capture()` the 2 x 81 launches are one graph replay."""
        self._weights_fresh = True
        if self.graph_refresh is not None:
            self.graph_refresh.replay()
            return
        for projs in self.blocks:
            self._refresh_block(projs)

    def zero_grads(self):
        for projs in self.blocks:
            for p in projs:
                p.gw.zero_()

    def _fwd_block_emit(self, projs, keep=False):
        T = self.T
        for p in projs:
            x = self.x_pool[p.name]
            if p.wq is None or p.wq.q is not p.q:
                p.wq = emit.WQ(p.N, p.K)
                p.wq.q, p.wq.qt = p.q, p.qt
            rq = emit.row_emit(x, emit.RowQ(T, p.K, self.device), None)
            p.cx = emit.col_emit(x, emit.ColQ(T, p.K, self.device), self.amax_use[p.lid, 0:1], self.amax_cur[p.lid, 0:1], self.rng)
            y = emit.mm_row_w(rq, p.wq, scale=True)
            p.y = y if keep else None

    def _bwd_block_emit(self, projs, keep=False, first=False, scatter=False):
        T = self.T
        alive = []          # operands the side stream still reads
        for p in reversed(projs):
            gy = self.gy_pool[p.name]
            use_x, use_g = self.amax_use[p.lid, 0:1], self.amax_use[p.lid, 1:2]
            rq = emit.row_emit(gy, emit.RowQ(T, p.N, self.device), self.rng, sr=self.emit_sr, salt=p.lid * 8 + 1)
            cg = emit.col_emit(gy, emit.ColQ(T, p.N, self.device), use_g, self.amax_cur[p.lid, 1:2], self.rng, sr=self.emit_sr,
                               salt=p.lid * 8 + 2)
            if self.wgrad_stream is not None:
                self.wgrad_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.wgrad_stream):
                    emit.mm_col(cg, p.cx, scale=True, amax_a=use_g, amax_b=use_x, out=p.gw, accumulate=not first,
                                owners=p.owners if scatter else None)
                alive.append(cg)
            gx = emit.mm_row_wt(rq, p.wq, scale=True)
            if self.wgrad_stream is None:
                emit.mm_col(cg, p.cx, scale=True, amax_a=use_g, amax_b=use_x, out=p.gw, accumulate=not first,
                            owners=p.owners if scatter else None)
            p.gx = gx if keep else None
        if self.wgrad_stream is not None:
            torch.cuda.current_stream().wait_stream(self.wgrad_stream)
        del alive

    def _fwd_block(self, projs, keep=False):
        if self.mode == "emit":
            return self._fwd_block_emit(projs, keep)
        # the block's amax words are cleared by one fill, so each projection is a kernel-to-kernel chain
        # amax -> quantizer -> GEMM with no fill node in between
        lo, hi = projs[0].lid, projs[-1].lid + 1
        self.am_words[0, lo:hi].zero_()
        for p in projs:
            y, p.am_x, p.qxt = linear_fwd(self.x_pool[p.name], p.q, keep_xt=True, signs=_RHT_SIGNS,
                                          am_out=self.am_words[0, p.lid:p.lid + 1])
            p.y = y if keep else None

    def _bwd_block(self, projs, keep=False, first=False, scatter=False):
        """`first`: the step's first microbatch overwrites dW instead of adding to it, so the
        gradients need no clearing pass.  `scatter` (`peer_reduce` stacks): the weight gradients are added into the
        owner ranks' slabs instead of this rank's buffer."""
        if self.mode == "emit":
            return self._bwd_block_emit(projs, keep, first, scatter)
        alive = []
        lo, hi = projs[0].lid, projs[-1].lid + 1
        self.am_words[1, lo:hi].zero_()
        for p in reversed(projs):
            sd = self.seeds[p.lid]
            gx, _ = linear_bwd(None, p.am_x, self.gy_pool[p.name], p.qt, sd[0:1], sd[1:2],
                               gw_out=p.gw, signs=_RHT_SIGNS, sr_mode=self.sr_mode, overwrite=first, qxt=p.qxt,
                               wgrad_stream=self.wgrad_stream, keep_alive=alive, am_out=self.am_words[1, p.lid:p.lid + 1],
                               gw_owners=p.owners if scatter else None)
            p.gx = gx if keep else None
        if self.wgrad_stream is not None:
            torch.cuda.current_stream().wait_stream(self.wgrad_stream)
        del alive

    def calibrate(self):
        """Emitter mode: two passes over all projections so that the delayed column scales come from observed
        amax values instead of the initial placeholder."""
        self.refresh_weights()
        for _ in range(2):
            for projs in self.blocks:
                self._fwd_block(projs)
            for projs in reversed(self.blocks):
                self._bwd_block(projs)
            self.roll_amax()
        self._calibrated = True

    def capture(self):
        """Capture each block's forward and backward into CUDA graphs sharing one memory pool."""
        self.refresh_weights()
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):          # warm-up outside capture (emitter mode: calibrates the delayed scales)
            for _ in range(2 if self.mode == "emit" else 1):
                for projs in self.blocks:
                    self._fwd_block(projs)
                for projs in reversed(self.blocks):
                    self._bwd_block(projs)
                if self.mode == "emit":
                    self.roll_amax()
        self._calibrated = True
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        pool = torch.cuda.graph_pool_handle()
        self.graphs_fwd, self.graphs_bwd, self.graphs_bwd_first = [], [], []
        for projs in self.blocks:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=pool):
                self._fwd_block(projs)
            self.graphs_fwd.append(g)
        # backward graphs run beside the gradient all-reduce: either keep `comm_sms` SMs out of the GEMM grids, or
        # (no budget) let every cluster draw even its first work item at run time, so that clusters which find
        # their SM taken by the collective and start late leave no item waiting for them
        lib = _lib.load()
        if self.comm_sms:
            sms = torch.cuda.get_device_properties(self.device).multi_processor_count
            lib.nvfp4_gemm_set_sm_budget(max(2, sms - self.comm_sms))
        elif self.group is not None or (torch.distributed.is_initialized() and torch.distributed.get_world_size() > 1):
            lib.nvfp4_gemm_set_scheduler(2)
        try:
            for first, store in ((True, self.graphs_bwd_first), (False, self.graphs_bwd)):
                for projs in reversed(self.blocks):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, pool=pool):
                        self._bwd_block(projs, first=first)
                    store.append(g)
            if self.peer_reduce:
                self.graphs_bwd_scatter = []
                for projs in reversed(self.blocks):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, pool=pool):
                        self._bwd_block(projs, scatter=True)
                    self.graphs_bwd_scatter.append(g)
        finally:
            lib.nvfp4_gemm_set_sm_budget(0)
            lib.nvfp4_gemm_set_scheduler(1)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, pool=pool):
            self.refresh_weights()           # buffers exist already: the in-place form is captured
        self.graph_refresh = g
        # per-block refresh graphs for the side stream: they run beside the backward graphs, so they get a pool of
        # their own (they allocate nothing: every output exists)
        self.graphs_refresh_blk = []
        for projs in self.blocks:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._refresh_block(projs)
            self.graphs_refresh_blk.append(g)
        torch.cuda.synchronize()

    def kernels_per_microbatch(self):
        """Kernels of this library launched per microbatch: fwd amax + tile quantizer + gemm;
        bwd amax + tile quantizer + 2 gemm (emitter mode: two emitters in place of amax + quantizer)."""
        return self.n_proj * (3 + 4)

    def microbatch(self, last, do_allreduce, first=False):
        """One forward + backward over all projections.  On the rank's last microbatch each block's
        weight gradients are all-reduced on the side stream right after its backward is enqueued."""
        self._bump_seeds()
        cur = torch.cuda.current_stream()
        if self.use_graphs and self.graphs_fwd is not None:
            for g in self.graphs_fwd:
                g.replay()
        else:
            for projs in self.blocks:
                self._fwd_block(projs)
        works = []
        nblk = len(self.blocks)
        scatter = self.peer_reduce and do_allreduce       # every microbatch of the step adds into the owners' slabs
        if scatter and first:
            cur.wait_event(self._peer_ready)              # all slabs are clear
        for i, projs in enumerate(reversed(self.blocks)):
            if self.use_graphs and self.graphs_bwd is not None:
                (self.graphs_bwd_scatter if scatter else self.graphs_bwd_first if first else self.graphs_bwd)[i].replay()
            else:
                self._bwd_block(projs, first=first, scatter=scatter)
            b = nblk - 1 - i
            reduce_now = last and do_allreduce and b in self.ar_after
            if reduce_now or (last and (self.overlap_refresh or self.after_reduce is not None)):
                ev = torch.cuda.Event()
                ev.record(cur)
                if reduce_now:
                    with torch.cuda.stream(self.comm_stream):
                        self.comm_stream.wait_event(ev)
                        if self.peer_reduce:
                            self._peer_finish_block(projs)
                        else:
                            allreduce_sum_([self.ar_after[b]], self.group)
                        ev = torch.cuda.Event()
                        ev.record()
                with torch.cuda.stream(self.refresh_stream):
                    self.refresh_stream.wait_event(ev)
                    if self.after_reduce is not None:
                        self.after_reduce(b, projs)
                    if self.overlap_refresh:
                        # the block's weights for the next step
                        if self.use_graphs and self.graphs_refresh_blk is not None:
                            self.graphs_refresh_blk[b].replay()
                        else:
                            self._refresh_block(projs)
        if self.mode == "emit":
            self.roll_amax()
        return works

    def step(self, n_micro, do_allreduce, before_microbatch=None):
        """One optimizer step's worth of this path: n_micro microbatches (the first overwrites dW, the others add),
        all-reduce, every weight re-quantized once (block by block behind the last microbatch's backward pass, or
        all at the start when `overlap_refresh` is off or the weights have never been quantized).  Leaves the summed
        FP32 gradients in `p.gw`.  `before_microbatch(m)`: called before each microbatch, e.g. to stage its input."""
        if self.mode == "emit" and not self._calibrated:
            self.calibrate()
        if not (self.overlap_refresh and self._weights_fresh):
            self.refresh_weights()           # otherwise the previous step re-quantized each block behind its backward
        if self.peer_reduce and do_allreduce:
            self._peer_begin_step()
        for m in range(n_micro):
            if before_microbatch is not None:
                before_microbatch(m)
            self.microbatch(last=(m == n_micro - 1), do_allreduce=do_allreduce, first=(m == 0))
        if do_allreduce or self.overlap_refresh or self.after_reduce is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
            torch.cuda.current_stream().wait_stream(self.refresh_stream)
