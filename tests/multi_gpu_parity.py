"""Run under torchrun with 2 or more ranks (one per GPU): the three ways of exchanging pooled rows and
gradients -- peer memory with the gradient push in two pieces, peer memory in one piece, NCCL all-to-all --
must leave every rank with bit-identical sketch state and tables after a few training steps.
Exit code 0 = identical on every rank."""
import datetime
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import numpy as np
import torch
import torch.distributed as dist


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))
    from cafe_b200.sharded import ShardedSKEmbedding
    from oracle.hotsketch import states_equal
    F, D, Bl, steps = 4 * world + 1, 32, 512, 6            # uneven field counts per rank on purpose
    cards = [3000 + 7919 * f for f in range(F)]
    models = {}
    for name, kw in (("pieces", dict(exchange="peer", pipeline_push=True)), ("whole", dict(exchange="peer", pipeline_push=False)),
                     ("nccl", dict(exchange="nccl"))):
        models[name] = ShardedSKEmbedding(cards, D, 0.02, 0.3, 1, 1, 1.0000005, device=dev, global_batch=Bl * world, lr=0.1,
                                          seed=5, **kw)
    rng = np.random.default_rng(100 + rank)
    bad = 0
    for step in range(steps):
        ids = torch.from_numpy(np.stack([np.minimum(rng.zipf(1.3, Bl) - 1, n - 1) for n in cards]).astype(np.int64)).to(dev)
        grad = None
        outs = {}
        for name, m in models.items():
            out = m(ids)
            if grad is None:
                grad = torch.from_numpy((rng.standard_normal(tuple(out.shape)) * 0.01).astype(np.float32)).to(dev)
            outs[name] = out.detach().clone()
            out.backward(grad)
        torch.cuda.synchronize()
        ref = models["nccl"]
        for name in ("pieces", "whole"):
            m = models[name]
            same_out = outs[name].numel() == outs["nccl"].numel() and torch.equal(outs[name].reshape(-1), outs["nccl"].reshape(-1))
            diffs = states_equal(ref.group.sketch.state(), m.group.sketch.state())
            same_w = torch.equal(ref.group.weight_high, m.group.weight_high) and all(
                torch.equal(a, b) for a, b in zip(ref.group.weight_hash, m.group.weight_hash))
            if diffs or not same_w:
                bad += 1
                print(f"rank {rank} step {step} {name}: state diffs {diffs[:3]} tables equal {same_w} outputs equal {same_out}", flush=True)
    t = torch.tensor([bad], device=dev)
    dist.all_reduce(t)
    if rank == 0:
        print("multi-GPU parity:", "identical" if int(t.item()) == 0 else f"{int(t.item())} mismatches", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(t.item()) == 0 else 1)


if __name__ == "__main__":
    main()
