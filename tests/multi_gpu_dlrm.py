"""Run under torchrun with 2 or more ranks (one per GPU): a data-parallel DLRM whose embedding fields are sharded over
the ranks (cafe_b200.dlrm_harness.run_data_parallel) trains on seeded synthetic data of the Kaggle shape (all 26
fields through the sketch), then a DCN of the Avazu shape (9 sketch fields sharded, 13 small plain tables replicated).
Checks on every rank: the losses are finite, the replicated parameters (MLPs, plain tables) are bit-identical on all
ranks after the last step, every owner's sketch took the global batch's lookups of its fields at every step, and the
loss falls.  Exit code 0 = all hold."""
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
    from cafe_b200 import dlrm_harness as H
    bad = []
    lines = []
    for shape, extra, steps, Bl in (("kaggle", ["--compress-rate", "0.001", "--hash-rate", "0.3", "--fused-interaction"], 80, 256),
                                    ("avazu", ["--model", "dcn", "--compress-rate", "0.1", "--hash-rate", "0.7"], 60, 512)):
        args = H.make_parser().parse_args(["--sketch-flag", "--sketch-alpha", "1.0000005", "--data-set", shape, "--mini-batch-size",
                                           str(Bl), "--nbatches", str(steps), "--warmup-batches", "10"] + extra)
        r = H.run_data_parallel(args)
        if not np.isfinite(r["losses"]).all():
            bad.append(f"{shape}: a loss is not finite")
        if not r["replicas_in_step"]:
            bad.append(f"{shape}: the dense replicas differ")
        if not r["loss_last"] < r["loss_first"]:
            bad.append(f"{shape}: loss did not fall: {r['loss_first']} -> {r['loss_last']}")
        want = steps * Bl * world * r["sketch_fields_this_rank"]
        if r["lookups_this_rank"] != want:
            bad.append(f"{shape}: sketch saw {r['lookups_this_rank']} lookups, expected {want}")
        lines.append(f"{shape} ({r['sketch_fields']} sketch + {r['plain_fields']} plain fields): loss {r['loss_first']:.4f} -> "
                     f"{r['loss_last']:.4f}, {r['samples_per_s']:.0f} samples/s")
    for b in bad:
        print(f"rank {rank}: {b}", flush=True)
    t = torch.tensor([len(bad)], device=dev)
    dist.all_reduce(t)
    if rank == 0:
        print(f"data-parallel training on {world} GPUs, fields sharded: " + "; ".join(lines) + ": " +
              ("in step" if int(t.item()) == 0 else f"{int(t.item())} problems"), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(t.item()) == 0 else 1)


if __name__ == "__main__":
    main()
