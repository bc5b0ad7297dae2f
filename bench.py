#!/usr/bin/env python
"""Benchmark of the CAFE compressed-embedding hot path (sketch + forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the hot path over one batch of the microbenchmark workload (26 fields x 40M
ids, Zipf 1.05, batch 65536 x 26 int64 ids, fp32 dim 128, N(0, 0.01) gradients, CAFE settings
compress 0.001 / hash-rate 0.3 / threshold 1 / alpha 1.0000005): fused query+gather forward, then
importance -> sketch insert -> migration -> scatter/SGD.  Prints ONE JSON line (rank 0).

`value` is measured with the ids already in HBM; `e2e` copies each step's ids from pinned host memory
and reads a slice of the result back.  `--impl reference` times the reference's own CPU
implementation of the same step (tricks/sketch.cpp compiled under oracle/_ref, or the C restatement
when that library is absent, plus PyTorch CPU embedding bags) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CR, HR, THR, ADJ, ALPHA = 0.001, 0.3, 1, 1, 1.0000005
DIM, BATCH, ZIPF_S, SEED = 128, 65536, 1.05, 2024
LR = 0.1
METRIC = "cafe_embedding_ids_per_s"
UNIT = "ids/s"
# algorithmic bytes per id of each kernel (R = 4*D bytes per row): what the kernel has to move
def alg_bytes(slot: str, D: int) -> float:
    R = 4 * D
    return {"embed_forward": 64 + 2 * R, "scatter_chunks": 3 * R + 8, "grad_norm": R + 4, "main_pass": 120,
            "lru_pass": 136, "row_sort": 16 * 3, "lookup_hash_sort": 16 * 3 * 2}.get(slot, 0.0)
FUSED_BYTES_PER_ID = lambda D: 192 + 5 * 4 * D   # query 64 + gather 2R + scatter 3R+8 + insert 120


def read_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples the SM clock and the throttle reasons of this rank's GPU while the timed region runs.

    NVML is read from a thread of this process and initialised before the warm-up, so that the timed region
    sees only the cheap per-sample queries and not one NVML start-up per rank against the driver while the steps
    are being launched.  Without the NVML module, rank 0 alone falls back to an nvidia-smi poller started ahead
    of the warm-up."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, uuid=None, allow_smi=True):
        self.idx, self.nv, self.h, self.proc = gpu_index, None, None, None
        self.samples, self.lines, self.on, self.t = [], [], False, None
        try:
            import pynvml
            pynvml.nvmlInit()
            h = None
            if uuid is not None:
                for cand in (f"GPU-{uuid}", str(uuid)):
                    try:
                        h = pynvml.nvmlDeviceGetHandleByUUID(cand.encode() if hasattr(cand, "encode") else cand)
                        break
                    except Exception:
                        h = None
            if h is None:
                h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
            self.nv, self.h = pynvml, h
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None
            if allow_smi:
                try:
                    self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms",
                                                  "50", "-i", str(gpu_index)], stdout=subprocess.PIPE,
                                                 stderr=subprocess.DEVNULL, text=True)
                    self.t = threading.Thread(target=self._read_smi, daemon=True)
                    self.t.start()
                except Exception:
                    self.proc = None

    def _read_smi(self):
        for line in self.proc.stdout:
            if self.on:
                self.lines.append(line.strip())

    def _poll(self):
        nv = self.nv
        while self.on:
            try:
                self.samples.append((float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)),
                                     int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))))
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        self.on = True
        if self.nv is not None:
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
        return self

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.06)
        self.on = False
        if self.nv is not None and self.t is not None:
            self.t.join(timeout=1)
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        if self.nv is not None and self.samples:
            nv = self.nv
            bits = [nv.nvmlClocksThrottleReasonHwSlowdown, nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                    nv.nvmlClocksThrottleReasonSwThermalSlowdown, nv.nvmlClocksThrottleReasonSwPowerCap]
            reasons = sorted({n for _, r in self.samples for n, b in zip(names, bits) if r & b})
            return {"sm_mhz": float(np.median([c for c, _ in self.samples])), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                    "samples": len(self.samples), "source": "nvml"}
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm),
                "source": "nvidia-smi"}


# -------------------------------------------------------------------------------------------------
# reference CPU path (the baseline): reference sketch library + PyTorch CPU embedding bags
# -------------------------------------------------------------------------------------------------
class CpuReferencePath:
    """The reference's own step on the host: query (C) -> two embedding_bag gathers + where
    (tricks/sk_embedding_bag.py:119-152) -> autograd backward -> importance (:178-189) -> batch_insert_val
    (C) -> guarded migration (:199-208) -> torch.optim.SGD on sparse gradients (dlrm_s_pytorch.py:1658)."""

    def __init__(self, cards, D, batch):
        import torch
        import torch.nn.functional as F
        from cafe_b200 import sizing
        from oracle import hotsketch as oh
        self.torch, self.Fn = torch, F
        self.cards, self.D, self.B = cards, D, batch
        self.hotn = sizing.hot_rows(sum(cards), CR, HR, D)
        self.hs = [sizing.hash_rows(n, CR, HR) for n in cards]
        self.off = sizing.field_offsets(cards)
        if oh.REF_SO.exists():
            self.sk, self.kind = oh.ReferenceSketch(self.hotn, THR, ADJ, ALPHA), "reference"
        else:
            self.sk, self.kind = oh.OracleSketch(self.hotn, THR, ADJ, ALPHA), "port"
        g = torch.Generator().manual_seed(1)
        self.wh = torch.nn.Parameter((torch.rand(self.hotn, D, generator=g) * 2 - 1) * float(np.sqrt(1 / max(cards))))
        self.wc = [torch.nn.Parameter((torch.rand(h, D, generator=g) * 2 - 1) * float(np.sqrt(1 / n)))
                   for h, n in zip(self.hs, cards)]
        self.opt = torch.optim.SGD([self.wh] + self.wc, lr=LR)
        self.offsets = torch.arange(batch)
        self.threads = torch.get_num_threads()

    def step(self, ids: np.ndarray, grad: "np.ndarray"):
        torch, F = self.torch, self.Fn
        outs, gids, qs = [], [], []
        for f in range(len(self.cards)):
            gid = ((ids[f].astype(np.int64) + self.off[f]) & 0xFFFFFFFF).astype(np.uint32)
            q = self.sk.batch_query(gid)
            dic = torch.from_numpy(np.abs(q.astype(np.int64)))
            mask = torch.from_numpy(q < 0).unsqueeze(1)
            hi = F.embedding_bag(dic % self.hotn, self.wh, self.offsets, sparse=True)
            lo = F.embedding_bag(dic % self.hs[f], self.wc[f], self.offsets, sparse=True)
            outs.append(torch.where(mask, hi, lo))
            gids.append(gid)
            qs.append(q)
        self.opt.zero_grad()
        torch.autograd.backward(outs, [grad[:, f] for f in range(len(outs))])
        for f in range(len(outs)):
            gn = torch.norm(grad[:, f], dim=1, p=2)
            imp = (gn * self.B / torch.sum(gn)).numpy()
            m = self.sk.batch_insert_val(gids[f], imp)
            q2 = self.sk.batch_query(gids[f])
            idx = np.nonzero((m != 0) & (q2 < 0))[0]
            if idx.size:
                with torch.no_grad():
                    self.wh[torch.from_numpy(-q2[idx].astype(np.int64))] = self.wc[f][torch.from_numpy(ids[f][idx] % self.hs[f])]
        self.opt.step()
        return outs


def run_reference(args, rank, world):
    if rank != 0:
        return
    import torch
    from cafe_b200 import synthetic as S
    cards = S.MICRO_CARDS
    B = args.cpu_batch
    path = CpuReferencePath(cards, DIM, B)
    F = len(cards)
    nb = 2
    ids = [S.batch_ids(cards, B, ZIPF_S, SEED, s) for s in range(nb)]
    grads = [torch.from_numpy(S.gradients(B, F, DIM, SEED, s)) for s in range(nb)]
    for s in range(args.warmup):
        path.step(ids[s % nb], grads[s % nb])
    t0 = time.perf_counter()
    for s in range(args.steps):
        path.step(ids[s % nb], grads[s % nb])
    dt = time.perf_counter() - t0
    v = args.steps * B * F / dt
    sample = f"{args.steps} steps of batch {B} x {F} fields after {args.warmup} warm-up steps (full batch is {BATCH})"
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(B, world=1),
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": path.threads, "kind": path.kind, "sample": sample,
                             "host_cpus": os.cpu_count()},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(batch, world):
    return {"workload": "hotsketch+skembeddingbag microbenchmark: 26 fields x 40M ids, Zipf(1.05) permuted, "
                        f"batch {batch} x 26 int64 ids, fp32 dim {DIM}, N(0,0.01) grads, compress 0.001, hash-rate 0.3, "
                        "threshold 1, alpha 1.0000005",
            "batch": batch, "fields": 26 * world, "dim": DIM, "ids_per_step": batch * 26 * world,
            "parallelism": (f"field-sharded x{world}: 26 fields (own sketch + tables) per GPU, global batch {batch}, pooled rows and "
                            "gradients exchanged through peer memory inside the gather / push kernels") if world > 1 else "single GPU",
            "l2": "per-step streams (ids, pooled output, gradients: 1.7 GB) exceed L2; no flush needed",
            "e2e_note": "ids come from pinned host memory every step and a slice of the pooled output is read back; "
                        "gradients stay on the device, where a training loop's dense backward produces them"}


def cpu_baseline_leg(args):
    """Bounded sample of the same workload through the reference's CPU path, on this host's cores."""
    import torch
    from cafe_b200 import synthetic as S
    cards = S.MICRO_CARDS
    B = args.cpu_batch
    path = CpuReferencePath(cards, DIM, B)
    F = len(cards)
    ids = [S.batch_ids(cards, B, ZIPF_S, SEED, s) for s in range(2)]
    grads = [torch.from_numpy(S.gradients(B, F, DIM, SEED, s)) for s in range(2)]
    warm, steps = 2, args.cpu_steps
    for s in range(warm):
        path.step(ids[s % 2], grads[s % 2])
    t0 = time.perf_counter()
    for s in range(steps):
        path.step(ids[s % 2], grads[s % 2])
    dt = time.perf_counter() - t0
    return {"value": steps * B * F / dt, "unit": UNIT, "cores": path.threads, "kind": path.kind,
            "sample": f"{steps} steps of batch {B} x {F} fields after {warm} warm-up steps (sketch single-threaded as in the "
                      f"reference, torch CPU ops on {path.threads} threads)", "ms_per_step": 1e3 * dt / steps,
            "host_cpus": os.cpu_count()}


# -------------------------------------------------------------------------------------------------
# our arm
# -------------------------------------------------------------------------------------------------
def run_ours(args, rank, world, local_rank):
    import torch
    import cafe_b200
    from cafe_b200 import profile as prof
    from cafe_b200 import synthetic as S

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        import datetime
        # a short timeout: a rank that stops (an exception, a mismatch) ends the job instead of hanging it
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))
    cards = S.MICRO_CARDS[:args.fields]
    F, D, B = len(cards), DIM, args.batch
    if world > 1:
        # weak scaling of a field-sharded model: every GPU brings its own copy of the workload's 26 fields
        # (26*N fields in all, rank g owns 26 of them with their sketch and tables), the global batch stays
        # 65536 samples, so each field still sees the batch the metric is quoted on and every rank serves
        # 26 x 65536 lookups per step, plus the exchange of its samples' rows with all other ranks
        from cafe_b200.sharded import ShardedSKEmbedding
        all_cards = cards * world
        offs = [(f // world) * 40_000_000 for f in range(len(all_cards))]   # distinct within each rank, < 2**31
        model = ShardedSKEmbedding(all_cards, D, CR, HR, THR, ADJ, ALPHA, device=dev, global_batch=B, lr=LR, seed=1,
                                   exchange=args.exchange, f_offsets=offs)
        step_fn, e2e_fn, ids_per_step = model.bench_closures(S, ZIPF_S, SEED)
    else:
        grp = cafe_b200.SKEmbeddingGroup(cards, D, CR, HR, THR, ADJ, ALPHA, device=dev, max_batch=B, lr=LR, seed=1)
        nb = 4
        host_ids = [torch.from_numpy(S.batch_ids(cards, B, ZIPF_S, SEED, s)).pin_memory() for s in range(nb)]
        dev_ids = [h.to(dev) for h in host_ids]
        g = torch.Generator(device=dev).manual_seed(SEED)
        grads = [torch.randn(B, F, D, device=dev, generator=g) * 0.01 for _ in range(2)]
        stage = torch.empty_like(dev_ids[0])
        res_host = torch.empty(16, F, D, dtype=torch.float32).pin_memory()
        ids_per_step = B * F

        def step_fn(s):
            out = grp(dev_ids[s % nb])
            out.backward(grads[s % 2])

        def e2e_fn(s):
            stage.copy_(host_ids[s % nb], non_blocking=True)
            out = grp(stage)
            out.backward(grads[s % 2])
            res_host.copy_(out.detach()[:16], non_blocking=True)
        h2d, d2h = host_ids[0].numel() * 8, res_host.numel() * 4

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, first):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(steps):
            fn(first + s)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device=dev)
            every = [torch.zeros_like(t) for _ in range(world)]
            dist.all_gather(every, t)
            timed.per_rank = [float(x.item()) for x in every]
            ms = max(timed.per_rank)
        return ms
    timed.per_rank = None

    try:
        uuid = torch.cuda.get_device_properties(dev).uuid
    except Exception:
        uuid = None
    clk = ClockSampler(local_rank, uuid, allow_smi=(rank == 0))   # set up ahead of the warm-up; samples only inside `with`
    for s in range(args.warmup):
        step_fn(s)
    barrier()
    l0 = prof.launch_count()
    with clk:   # the clock samples cover both timed regions (resident inputs and end to end)
        ms = timed(step_fn, args.steps, args.warmup)
        step_ms_per_rank = [round(x / args.steps, 3) for x in timed.per_rank] if timed.per_rank else None
        launches = prof.launch_count() - l0
        total_ids = ids_per_step * (world if world > 1 else 1)
        value = args.steps * total_ids / (ms / 1e3)

        # end to end: ids from pinned host memory each step, result slice read back
        for s in range(3):
            e2e_fn(s)
        ms_e2e = timed(e2e_fn, args.steps, 0)
        e2e_value = args.steps * total_ids / (ms_e2e / 1e3)
    clocks = clk.summary()

    # per-kernel times, live, with CUDA events on the launching stream (every rank runs the pass: the steps
    # contain collectives; rank 0 reports its own kernels)
    prof.read()
    prof.enable(True)
    ms_prof = timed(step_fn, args.steps, args.warmup + args.steps)
    slots = prof.read()
    prof.enable(False)
    rank_info = None
    if dist is not None:
        # how evenly the ranks are loaded: every rank's own kernel time per step (sum of its per-kernel times)
        mine = torch.tensor([sum(v[0] for v in slots.values()) / args.steps], device=dev)
        allr = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        names = sorted(slots.keys())
        vec = torch.tensor([slots[k][0] / args.steps for k in names], device=dev, dtype=torch.float32)
        allv = [torch.zeros_like(vec) for _ in range(world)]
        dist.all_gather(allv, vec)
        per_slot = {k: [round(float(allv[r][i].item()), 3) for r in range(world)] for i, k in enumerate(names)
                    if max(float(allv[r][i].item()) for r in range(world)) >= 0.05}
        rank_info = {"phase_ms_per_rank": per_slot, "step_ms": step_ms_per_rank, "own_kernel_ms_per_step": [round(float(t.item()), 3) for t in allr],
                     "host_cpus": len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else os.cpu_count()}
    line = None
    if rank == 0:
        peak, peak_kind = read_peaks()
        phases = {k: {"ms_per_step": v[0] / args.steps, "launches_per_step": v[1] / args.steps}
                  for k, v in slots.items() if v[1] > 0}
        cand = {k: v for k, v in slots.items() if alg_bytes(k, D) > 0 and v[1] > 0}
        # the sketch passes run in three modes (all buckets / later rounds / final pass) that are timed in slots of
        # their own: the kernel is ranked by their sum and reported on its all-bucket launches
        group = {"main_pass": ("main_pass", "main_pass_later_rounds", "main_pass_final"),
                 "lru_pass": ("lru_pass", "lru_pass_later_rounds")}
        rank = lambda k: sum(slots[g][0] for g in group.get(k, (k,)) if g in slots)
        top = max(cand, key=rank) if cand else None
        roof = None
        if top:
            per_launch_ms = cand[top][0] / cand[top][1]
            # lookups one launch processes: the per-step kernels see every lookup of the step once; the
            # sketch passes run once or more per job over that job's window, and all windows of a step
            # add up to the step's lookups, so an average launch covers ids_per_step / launches_per_step
            launches_per_step = cand[top][1] / args.steps
            units = ids_per_step / max(1.0, launches_per_step)
            ach = alg_bytes(top, D) * units / (per_launch_ms / 1e3) / 1e9
            traffic = None
            tp = ROOT / "profiles" / "traffic.json"
            if tp.exists():
                try:
                    per_id = json.loads(tp.read_text()).get(top, {}).get("dram_bytes_per_id")
                    traffic = per_id * units if per_id else None
                except Exception:
                    traffic = None
            roof = {"bound": "hbm", "kernel": top, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                    "traffic": traffic, "peak_kind": peak_kind, "alg_bytes_per_id": alg_bytes(top, D),
                    "ms_per_launch": per_launch_ms, "ids_per_launch": units,
                    "fused_path": {"alg_bytes_per_id": FUSED_BYTES_PER_ID(D),
                                   "achieved": FUSED_BYTES_PER_ID(D) * total_ids / (ms / args.steps / 1e3) / 1e9 / max(world, 1),
                                   "frac": FUSED_BYTES_PER_ID(D) * total_ids / (ms / args.steps / 1e3) / 1e9 / max(world, 1) / peak}}
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic", "config": workload_config(B, world),
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d if world == 1 else model.h2d_bytes,
                        "d2h_bytes_per_step": d2h if world == 1 else model.d2h_bytes, "ms_per_step": ms_e2e / args.steps},
                "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "phases": phases,
                "phases_note": "per-kernel CUDA-event times of a separate pass with the side-stream overlap switched off",
                "ms_per_step_profiled": ms_prof / args.steps}
        if rank_info is not None:
            line["ranks"] = rank_info
        if world == 1:
            line["sketch"] = {k: v for k, v in grp.sketch.stats().items()}
        if world == 1 and not args.no_cpu_baseline:
            try:
                line["cpu_baseline"] = cpu_baseline_leg(args)
            except Exception as e:  # the baseline is informative; never lose the GPU number to it
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "unavailable", "sample": repr(e)}
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH, help="samples per GPU per step")
    ap.add_argument("--cpu-batch", type=int, default=16384, help="batch of the CPU baseline sample")
    ap.add_argument("--cpu-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--fields", type=int, default=26, help="use only the first N fields of the workload (experiments)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="multi-GPU exchange of pooled rows / gradients")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
