"""Run under torchrun with 2 or more ranks (one per GPU).  Two checks after every training step:

  1. per-shard parity: every rank drives a CPU oracle (sequential sketch + numpy module step) over ITS OWN fields
     with the global field offsets, fed the global batch's ids and gradients gathered from all ranks; the rank's
     sketch state must equal the oracle's bit for bit, its tables within 1e-5, and the pooled rows that every
     consumer received from this owner must equal the oracle's forward;
  2. the three ways of exchanging pooled rows and gradients -- peer memory with the gradient push in two pieces,
     peer memory in one piece, NCCL all-to-all -- must leave bit-identical state, tables and outputs.

Exit code 0 = both hold on every rank.  If CAFE_PARITY_REPORT names a file, rank 0 writes its one-line result there."""
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
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    from cafe_b200 import sizing
    from cafe_b200.sharded import ShardedSKEmbedding
    from oracle.hotsketch import OracleSketch, states_equal
    from oracle.module_oracle import ModuleOracle
    F, D, Bl, steps = 4 * world + 1, 32, 512, 6            # uneven field counts per rank on purpose
    cards = [3000 + 7919 * f for f in range(F)]
    models = {}
    for name, kw in (("pieces", dict(exchange="peer", pipeline_push=True)), ("whole", dict(exchange="peer", push="whole")),
                     ("norms", dict(exchange="peer", push="norms_first")), ("nccl", dict(exchange="nccl"))):
        models[name] = ShardedSKEmbedding(cards, D, 0.02, 0.3, 1, 1, 1.0000005, device=dev, global_batch=Bl * world, lr=0.1,
                                          seed=5, **kw)
    ref = models["nccl"]
    plan, grp = ref.plan, ref.group
    mine = plan.local_fields
    offs = sizing.field_offsets(cards)
    assert grp.f_offsets == [offs[f] for f in mine], "shards must keep the global field offsets"
    sk = OracleSketch(grp.hotn, 1, 1, 1.0000005)
    orc = ModuleOracle(sk, grp.weight_high.detach().cpu().numpy(), [w.detach().cpu().numpy() for w in grp.weight_hash],
                       grp.f_offsets, grp.hash_sizes)
    rng = np.random.default_rng(100 + rank)
    bad = 0

    def complain(msg):
        nonlocal bad
        bad += 1
        print(f"rank {rank}: {msg}", flush=True)

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
        # ---- the oracle's view of this shard: global batch of the rank's own fields
        all_ids = [torch.empty_like(ids) for _ in range(world)]
        dist.all_gather(all_ids, ids)
        own_ids = torch.cat([a[mine] for a in all_ids], dim=1).cpu().numpy()            # [F_g, B_global], slices by rank
        all_grad = [torch.empty_like(grad) for _ in range(world)]
        dist.all_gather(all_grad, grad)
        g_own = torch.cat([plan.blocks(a, Bl, D)[plan.rank] for a in all_grad], dim=0).contiguous()   # [B_global, F_g, D]
        all_out = [torch.empty_like(outs["nccl"]) for _ in range(world)]
        dist.all_gather(all_out, outs["nccl"])
        pooled_ref = orc.forward(own_ids)                                                # [B_global, F_g, D]
        for q in range(world):
            got = plan.blocks(all_out[q], Bl, D)[plan.rank].cpu().numpy()
            if not np.allclose(got, pooled_ref[q * Bl:(q + 1) * Bl], rtol=1e-5, atol=1e-7):
                complain(f"step {step}: pooled rows delivered to rank {q} differ from the oracle's forward")
        Fg, Bg = len(mine), world * Bl
        imp = grp._fields.importance(g_own, D, Fg * D, Bg).view(Fg, Bg).cpu().numpy()
        orc.backward(own_ids, g_own.cpu().numpy(), grp.lr, importance=imp)
        diffs = states_equal(sk.state(), grp.sketch.state())
        if diffs:
            complain(f"step {step}: sketch state differs from the per-shard oracle: {diffs[:4]}")
        if not np.allclose(grp.weight_high.detach().cpu().numpy(), orc.wh, rtol=1e-5, atol=1e-7):
            complain(f"step {step}: hot table differs from the per-shard oracle")
        for j in range(Fg):
            if not np.allclose(grp.weight_hash[j].detach().cpu().numpy(), orc.wc[j], rtol=1e-5, atol=1e-7):
                complain(f"step {step}: hash table of field {mine[j]} differs from the per-shard oracle")
        # ---- the exchange variants against each other
        for name in ("pieces", "whole", "norms"):
            m = models[name]
            same_out = outs[name].numel() == outs["nccl"].numel() and torch.equal(outs[name].reshape(-1), outs["nccl"].reshape(-1))
            diffs = states_equal(ref.group.sketch.state(), m.group.sketch.state())
            same_w = torch.equal(ref.group.weight_high, m.group.weight_high) and all(
                torch.equal(a, b) for a, b in zip(ref.group.weight_hash, m.group.weight_hash))
            if diffs or not same_w or not same_out:
                complain(f"step {step} {name}: state diffs {diffs[:3]} tables equal {same_w} outputs equal {same_out}")
    t = torch.tensor([bad], device=dev)
    dist.all_reduce(t)
    if rank == 0:
        verdict = "identical" if int(t.item()) == 0 else f"{int(t.item())} mismatches"
        line = f"multi-GPU parity on {world} GPUs ({steps} steps, per-shard oracle and four exchange variants): {verdict}"
        print(line, flush=True)
        if os.environ.get("CAFE_PARITY_REPORT"):
            Path(os.environ["CAFE_PARITY_REPORT"]).write_text(line + "\n")
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(t.item()) == 0 else 1)


if __name__ == "__main__":
    main()
