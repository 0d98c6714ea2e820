"""One rank of the 2-GPU check of the reduce-scatter in the weight-gradient GEMM epilogues (launched by
test_gpu_peer_reduce.py through torch.distributed.run): a stack that reduces its gradients through peer memory
must leave the same sums as the same stack with NCCL's all-reduce, step after step, eager and graph-replayed."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nvfp4_training_b200 import _lib  # noqa: E402
from nvfp4_training_b200.stack import LinearStack, StackConfig  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    cfg = StackConfig(vocab=8192, layers=2)
    ok = True
    worst = 0.0
    for mode in ("tensor", "emit"):
        for graphs in (False, True):
            kw = dict(seed=3, input_seed=100 + rank, use_graphs=graphs, mode=mode)
            ref = LinearStack(cfg, 1024, dev, peer_reduce=False, **kw)
            peer = LinearStack(cfg, 1024, dev, peer_reduce=True, **kw)
            if graphs:
                ref.capture()
                peer.capture()
            else:
                ref.refresh_weights()
                peer.refresh_weights()
                if mode == "emit":
                    ref.calibrate()
                    peer.calibrate()
            peer.micro_count = ref.micro_count
            for step in range(3):
                n_micro = 1 + step % 2
                ref.step(n_micro, do_allreduce=True)
                peer.step(n_micro, do_allreduce=True)
                torch.cuda.synchronize()
                for br, bp in zip(ref.blocks, peer.blocks):
                    for pr, pp in zip(br, bp):
                        err = ((pr.gw - pp.gw).abs().max() / pr.gw.abs().max()).item()
                        worst = max(worst, err)
                        if not (err <= 2e-6) or not bool(pr.gw.abs().max() > 0):
                            ok = False
                            print(f"rank {rank}: {mode} graphs={graphs} step {step} {pr.name}: err {err}", flush=True)
            # without the exchange the same stack leaves this rank's own gradients, as before
            ref.step(1, do_allreduce=False)
            peer.step(1, do_allreduce=False)
            torch.cuda.synchronize()
            for br, bp in zip(ref.blocks, peer.blocks):
                for pr, pp in zip(br, bp):
                    if not torch.equal(pr.gw, pp.gw):
                        ok = False
                        print(f"rank {rank}: {mode} graphs={graphs}: local gradients differ ({pr.name})", flush=True)
            _lib.check_status()
            dist.barrier()              # no rank lets go of its buffers while another may still add into them
            torch.cuda.synchronize()
            del ref, peer
            torch.cuda.empty_cache()
    flag = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print(f"worst relative difference {worst:.3g}", flush=True)
        print("PEER_REDUCE_OK" if flag.item() == 1.0 else "PEER_REDUCE_FAILED", flush=True)
    dist.destroy_process_group()
    return 0 if flag.item() == 1.0 else 1


if __name__ == "__main__":
    sys.exit(main())
