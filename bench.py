#!/usr/bin/env python
"""Benchmark of the CAFE compressed-embedding hot path (sketch + forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload auto|micro|cfg3|weak26]

One step = one pass of the hot path over one batch: fused query+gather forward, then importance ->
sketch insert -> migration -> scatter/SGD.  Every step gets a batch of ids of its own (nothing is
replayed) and a gradient buffer of its own.  Prints ONE JSON line (rank 0).

Workloads (`--workload auto` picks `micro` on one GPU and `cfg3` on several):
  micro   the HotSketch + SKEmbeddingBag microbenchmark: 26 fields x 40M ids, Zipf 1.05, batch 65536 x 26
          int64 ids, fp32 dim 128, N(0, 0.01) gradients, compress 0.001 / hash-rate 0.3 / threshold 1 /
          alpha 1.0000005;
  cfg3    the Terabyte-shaped drifting workload: 26 fields with the Criteo-Terabyte cardinalities sharded by
          field (round robin) over the GPUs, global batch 65536, dim 128, compress 0.0001 / hash-rate 0.2,
          Zipf exponent drifting 1.05 -> 1.2 over 10k workload steps with 5 % of the ids re-permuted every
          1k workload steps; one bench step advances the workload by --drift-stride steps;
  weak26  every GPU brings 26 microbenchmark fields of its own (26*N fields), global batch 65536.

`value` is measured with the ids already in HBM; `e2e` copies each step's ids from pinned host memory
and reads a slice of the result back, on a sketch that starts from the same state and sees the same
batches as `value`.  `--impl reference` times the reference's own CPU implementation of the same step on
the same workload (tricks/sketch.cpp compiled under oracle/_ref, or the C restatement when that library
is absent, plus PyTorch CPU embedding bags) on all host cores.
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

THR, ADJ, ALPHA = 1, 1, 1.0000005
DIM, BATCH, SEED = 128, 65536, 2024
LR = 0.1
METRIC = "cafe_embedding_ids_per_s"
UNIT = "ids/s"
# Algorithmic bytes per id of each kernel (R = 4*D bytes per row): what the kernel has to move.  `u` is the share of
# lookups that name a table row no earlier lookup of the step names (measured on the last timed batch): a row that
# many lookups share has to be read once by the gather and read and written once by the scatter, while every lookup
# has its own pooled row to write and its own gradient row to read.
def alg_bytes(slot: str, D: int, u: float = 1.0) -> float:
    R = 4 * D
    return {"embed_forward": 64 + R + u * R, "scatter_chunks": R + 8 + 2 * u * R, "grad_norm": R + 4, "main_pass": 120,
            "lru_pass": 136, "row_sort": 16 * 3, "lookup_hash_sort": 16 * 3 * 2}.get(slot, 0.0)
FUSED_BYTES_PER_ID = lambda D, u=1.0: 192 + (2 + 3 * u) * 4 * D   # query 64 + gather R+uR + scatter R+8+2uR + insert 120


def unique_row_share(codes) -> float:
    """codes int32 [F, B] from SKEmbeddingGroup.row_codes: distinct table rows / lookups (hot rows are shared by all
    fields, hash rows belong to their field)."""
    import torch
    F = codes.shape[0]
    c = codes.to(torch.int64)
    field = torch.arange(F, device=codes.device, dtype=torch.int64)[:, None]
    key = torch.where(c < 0, c, (field << 32) | c)
    return float(torch.unique(key).numel()) / max(1, key.numel())


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
        self.samples, self.lines, self.on, self.t, self.stop = [], [], False, None, False
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
        while not self.stop:
            if self.on:
                try:
                    self.samples.append((float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)),
                                         int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))))
                except Exception:
                    pass
            time.sleep(0.002)

    # `with sampler:` may be entered several times: samples are taken only inside, one polling thread serves all
    def __enter__(self):
        self.on = True
        if self.nv is not None and self.t is None:
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
        return self

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.06)
        self.on = False

    def close(self):
        self.stop = True
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
# workloads
# -------------------------------------------------------------------------------------------------
class Workload:
    """One named workload: field cardinalities, CAFE sizing rates and the id stream (a batch per step)."""

    def __init__(self, name: str, world: int, stride: int):
        from cafe_b200 import sizing, synthetic as S
        self.name, self.world, self.stride, self.S = name, world, stride, S
        if name == "micro":
            self.cards, self.cr, self.hr = list(S.MICRO_CARDS), 0.001, 0.3
            self.offsets = sizing.field_offsets(self.cards)
        elif name == "cfg3":
            self.cards, self.cr, self.hr = list(S.TERABYTE_CARDS), 0.0001, 0.2
            self.offsets = sizing.field_offsets(self.cards)
        elif name == "weak26":
            self.cards, self.cr, self.hr = list(S.MICRO_CARDS) * world, 0.001, 0.3
            # 26*N*40M ids do not fit 31 bits: offsets are distinct within each rank only (ranks share no state)
            self.offsets = [(f // world) * 40_000_000 for f in range(len(self.cards))]
        else:
            raise ValueError(name)
        self.F = len(self.cards)
        self.scaling = "weak" if name == "weak26" or world == 1 else "strong"

    def ids(self, step: int, batch: int, rank: int = 0) -> np.ndarray:
        """ids [F, batch] of the GLOBAL batch of `step` (weak26: of this rank's slice)."""
        S = self.S
        if self.name == "micro":
            return S.batch_ids(self.cards, batch, 1.05, SEED, step)
        if self.name == "cfg3":
            return S.drift_batch_ids(self.cards, batch, SEED, step * self.stride)
        return S.batch_ids(self.cards, batch, 1.05, SEED + 7919 * rank, step)

    def config(self, batch: int) -> dict:
        w = self.world
        if self.name == "micro":
            what = ("hotsketch+skembeddingbag microbenchmark: 26 fields x 40M ids, Zipf(1.05) permuted, "
                    f"batch {batch} x 26 int64 ids, fp32 dim {DIM}, N(0,0.01) grads, compress 0.001, hash-rate 0.3, "
                    "threshold 1, alpha 1.0000005; a fresh id batch and gradient every step")
            par = "single GPU"
        elif self.name == "cfg3":
            what = ("Terabyte-shaped drifting workload: 26 fields with the Criteo-Terabyte cardinalities, "
                    f"global batch {batch} x 26 int64 ids, fp32 dim {DIM}, N(0,0.01) grads, compress 0.0001, hash-rate 0.2, "
                    "threshold 1, alpha 1.0000005; Zipf exponent 1.05 -> 1.2 over 10k workload steps, 5% of ids "
                    f"re-permuted every 1k workload steps, one bench step = {self.stride} workload steps; a fresh id "
                    "batch and gradient every step")
            par = (f"field-sharded x{w}: 26 fields round robin over the GPUs (own sketch + tables per GPU), pooled rows and "
                   "gradients exchanged through peer memory inside the gather / push kernels") if w > 1 else "single GPU"
        else:
            what = (f"26 microbenchmark fields per GPU ({26 * w} fields x 40M ids, Zipf 1.05), global batch {batch}, fp32 dim "
                    f"{DIM}, compress 0.001, hash-rate 0.3, threshold 1; a fresh id batch and gradient every step")
            par = f"field-sharded x{w}: 26 fields (own sketch + tables) per GPU, exchange through peer memory"
        return {"workload": what, "name": self.name, "batch": batch, "fields": self.F, "dim": DIM,
                "ids_per_step": batch * self.F, "parallelism": par,
                "l2": "per-step streams (ids, pooled output, gradients: 1.7 GB) exceed L2; no flush needed",
                "e2e_note": "ids come from pinned host memory every step (the copy of the next step's ids runs on a copy stream "
                            "beside the current step) and a slice of the pooled output is read back; gradients stay on the "
                            "device, where a training loop's dense backward produces them"}


def generate_batches(wl: Workload, steps, batch: int, rank: int = 0, cols=None):
    """[np.ndarray [F, cols]] for the given workload steps, generated by a few host threads."""
    from concurrent.futures import ThreadPoolExecutor

    def one(s):
        a = wl.ids(s, batch, rank)
        return np.ascontiguousarray(a if cols is None else a[:, cols[0]:cols[1]])
    with ThreadPoolExecutor(max_workers=max(1, min(8, (os.cpu_count() or 2) // 2))) as ex:
        return list(ex.map(one, steps))


# -------------------------------------------------------------------------------------------------
# reference CPU path (the baseline): reference sketch library + PyTorch CPU embedding bags
# -------------------------------------------------------------------------------------------------
class CpuReferencePath:
    """The reference's own step on the host: query (C) -> two embedding_bag gathers + where
    (tricks/sk_embedding_bag.py:119-152) -> autograd backward -> importance (:178-189) -> batch_insert_val
    (C) -> guarded migration (:199-208) -> torch.optim.SGD on sparse gradients (dlrm_s_pytorch.py:1658)."""

    def __init__(self, wl: Workload, D, batch):
        import torch
        import torch.nn.functional as F
        from cafe_b200 import sizing
        from oracle import hotsketch as oh
        # torch.distributed.run exports OMP_NUM_THREADS=1: the baseline gets every host core it may use regardless
        ncpu = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        torch.set_num_threads(max(1, ncpu))
        self.torch, self.Fn = torch, F
        cards = wl.cards
        self.cards, self.D, self.B = cards, D, batch
        self.hotn = sizing.hot_rows(sum(cards), wl.cr, wl.hr, D)
        self.hs = [sizing.hash_rows(n, wl.cr, wl.hr) for n in cards]
        self.off = wl.offsets
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

    def step(self, ids: np.ndarray, grad):
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


def time_cpu_path(wl: Workload, batch: int, warm: int, steps: int):
    """(ids/s, ms per step, path) of the reference's CPU step over fresh batches 0 .. warm+steps-1."""
    import torch
    path = CpuReferencePath(wl, DIM, batch)
    ids = generate_batches(wl, range(warm + steps), batch)
    ng = min(warm + steps, 4)   # gradients: a few distinct buffers (the host holds 0.9 GB each at full batch)
    gg = torch.Generator().manual_seed(SEED)
    grads = [torch.randn(batch, wl.F, DIM, generator=gg) * 0.01 for _ in range(ng)]
    for s in range(warm):
        path.step(ids[s], grads[s % ng])
    t0 = time.perf_counter()
    for s in range(warm, warm + steps):
        path.step(ids[s], grads[s % ng])
    dt = time.perf_counter() - t0
    return steps * batch * wl.F / dt, 1e3 * dt / steps, path


def run_reference(args, rank, world):
    if rank != 0:
        return
    wl = Workload(args.workload, world, args.drift_stride)
    B = args.cpu_batch
    v, ms, path = time_cpu_path(wl, B, args.warmup, args.steps)
    sample = (f"{args.steps} steps of batch {B} x {wl.F} fields after {args.warmup} warm-up steps, a fresh batch every step "
              f"(sketch single-threaded as in the reference, torch CPU ops on {path.threads} threads)")
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": wl.scaling,
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": wl.config(B),
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": path.threads, "kind": path.kind, "sample": sample,
                             "host_cpus": os.cpu_count()},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


def cpu_baseline_leg(args, wl):
    """Bounded sample of the same workload through the reference's CPU path, on this host's cores."""
    warm, steps = 1, args.cpu_steps
    v, ms, path = time_cpu_path(wl, args.cpu_batch, warm, steps)
    return {"value": v, "unit": UNIT, "cores": path.threads, "kind": path.kind,
            "sample": f"{steps} steps of batch {args.cpu_batch} x {wl.F} fields after {warm} warm-up step, a fresh batch every "
                      f"step (sketch single-threaded as in the reference, torch CPU ops on {path.threads} threads)",
            "ms_per_step": ms, "host_cpus": os.cpu_count()}


# -------------------------------------------------------------------------------------------------
# our arm
# -------------------------------------------------------------------------------------------------
class SingleGpuRun:
    """All fields of the workload on one GPU behind SKEmbeddingGroup."""

    def __init__(self, wl, B, dev):
        import cafe_b200
        self.grp = cafe_b200.SKEmbeddingGroup(wl.cards, DIM, wl.cr, wl.hr, THR, ADJ, ALPHA, device=dev, max_batch=B, lr=LR,
                                              seed=1, f_offsets=wl.offsets)
        self.out = None

    def step(self, ids_dev, grad):
        self.out = self.grp(ids_dev)
        self.out.backward(grad)

    def result_slice(self):
        return self.out.detach()[:16]

    def grad_shape(self, B, wl):
        return (B, wl.F, DIM)

    def stats(self):
        return self.grp.sketch.stats()


class ShardedRun:
    """Fields sharded over the ranks behind ShardedSKEmbedding; every rank feeds its slice of the global batch."""

    def __init__(self, wl, B, dev, exchange):
        from cafe_b200.sharded import ShardedSKEmbedding
        self.model = ShardedSKEmbedding(wl.cards, DIM, wl.cr, wl.hr, THR, ADJ, ALPHA, device=dev, global_batch=B, lr=LR, seed=1,
                                        exchange=exchange, f_offsets=wl.offsets)
        self.out = None

    def step(self, ids_dev, grad):
        self.out = self.model(ids_dev)
        self.out.backward(grad)

    def result_slice(self):
        return self.out.detach().reshape(-1)[:16 * DIM]

    def grad_shape(self, B, wl):
        return (B // wl.world * wl.F * DIM,)

    def stats(self):
        return self.model.group.sketch.stats()


def run_ours(args, rank, world, local_rank):
    import torch
    from cafe_b200 import profile as prof

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        import datetime
        # a short timeout: a rank that stops (an exception, a mismatch) ends the job instead of hanging it
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    wl = Workload(args.workload, world, args.drift_stride)
    B, W, K = args.batch, args.warmup, args.steps
    Bl = B // world
    cols = None if (world == 1 or wl.name == "weak26") else (rank * Bl, (rank + 1) * Bl)
    gen_batch = Bl if wl.name == "weak26" else B
    # steps 0 .. W+K-1 feed the warm-up and the timed region (the end-to-end measurement sees the same ones on a
    # sketch built anew); W+K .. W+2K-1 feed the per-kernel timing pass
    host_ids = [torch.from_numpy(a).pin_memory() for a in generate_batches(wl, range(W + 2 * K), gen_batch, rank, cols)]
    dev_ids = [h.to(dev) for h in host_ids]
    make = (lambda: SingleGpuRun(wl, B, dev)) if world == 1 else (lambda: ShardedRun(wl, B, dev, args.exchange))
    run = make()
    g = torch.Generator(device=dev).manual_seed(SEED + rank)
    ng = min(W + K, 32)
    grads = [torch.randn(run.grad_shape(B, wl), device=dev, generator=g) * 0.01 for _ in range(ng)]
    # end to end: two staging buffers and a copy stream, so that the copy of step s+1's ids from pinned host memory
    # runs beside step s (what a prefetching loader does); every step's copy lies inside the timed region
    stages = [torch.empty_like(dev_ids[0]) for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=dev)
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    res_host = torch.empty(16 * (wl.F if world == 1 else 1) * DIM, dtype=torch.float32).pin_memory()
    ids_per_step = B * wl.F                       # whole job, all ranks together
    h2d, d2h = host_ids[0].numel() * 8 * world, res_host.numel() * 4 * world

    def step_fn(s):
        run.step(dev_ids[s], grads[s % ng])

    def e2e_prefetch(s):
        b = s % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[b])        # the step that last read this buffer has finished its forward
            stages[b].copy_(host_ids[s], non_blocking=True)
            copied[b].record(copy_stream)

    def e2e_fn(s):
        main = torch.cuda.current_stream()
        if s == e2e_fn.first:
            e2e_prefetch(s)
        main.wait_event(copied[s % 2])
        if s + 1 < len(host_ids):
            e2e_prefetch(s + 1)
        run.step(stages[s % 2], grads[s % ng])
        consumed[s % 2].record(main)
        res_host.copy_(run.result_slice().reshape(-1), non_blocking=True)
    e2e_fn.first = W

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
    for s in range(W):
        step_fn(s)
    barrier()
    st0 = run.stats()
    l0 = prof.launch_count()
    with clk:   # the clock samples cover the two timed regions (resident inputs, end to end) and nothing else
        ms = timed(step_fn, K, W)
    step_ms_per_rank = [round(x / K, 3) for x in timed.per_rank] if timed.per_rank else None
    launches = prof.launch_count() - l0
    st1 = run.stats()
    value = K * ids_per_step / (ms / 1e3)
    # end to end: the same batches on a sketch and tables built anew and warmed up the same way, ids from pinned
    # host memory each step, a slice of the result read back
    run = None
    torch.cuda.empty_cache()
    run = make()
    for s in range(W):
        step_fn(s)
    with clk:
        ms_e2e = timed(e2e_fn, K, W)
    e2e_value = K * ids_per_step / (ms_e2e / 1e3)
    clocks = clk.summary()
    clk.close()

    # per-kernel times, live, with CUDA events on the launching stream (every rank runs the pass: the steps
    # contain collectives; rank 0 reports its own kernels)
    prof.read()
    prof.enable(True)
    ms_prof = timed(step_fn, K, W + K)
    slots = prof.read()
    prof.enable(False)
    rank_info = None
    if dist is not None:
        # how evenly the ranks are loaded: every rank's own kernel time per step (sum of its per-kernel times)
        mine = torch.tensor([sum(v[0] for v in slots.values()) / K], device=dev)
        allr = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        names = sorted(slots.keys())
        vec = torch.tensor([slots[k][0] / K for k in names], device=dev, dtype=torch.float32)
        allv = [torch.zeros_like(vec) for _ in range(world)]
        dist.all_gather(allv, vec)
        per_slot = {k: [round(float(allv[r][i].item()), 3) for r in range(world)] for i, k in enumerate(names)
                    if max(float(allv[r][i].item()) for r in range(world)) >= 0.05}
        rank_info = {"phase_ms_per_rank": per_slot, "step_ms": step_ms_per_rank,
                     "own_kernel_ms_per_step": [round(float(t.item()), 3) for t in allr],
                     "host_cpus": len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else os.cpu_count()}
    single_ref = None
    if dist is not None and wl.name == "cfg3" and not args.no_single_ref:
        # strong-scaling context: the same workload un-sharded on ONE GPU (rank 0; the others wait), same steps
        if rank == 0:
            wl1 = Workload("cfg3", 1, args.drift_stride)
            ids1 = [torch.from_numpy(a).to(dev) for a in generate_batches(wl1, range(W + K), B)]
            one = SingleGpuRun(wl1, B, dev)
            g1 = [torch.randn(B, wl1.F, DIM, device=dev, generator=g) * 0.01 for _ in range(min(W + K, 8))]
            for s in range(W):
                one.step(ids1[s], g1[s % len(g1)])
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for s in range(W, W + K):
                one.step(ids1[s], g1[s % len(g1)])
            e1.record()
            torch.cuda.synchronize()
            ms1 = e0.elapsed_time(e1)
            single_ref = {"value": K * ids_per_step / (ms1 / 1e3), "unit": UNIT, "ms_per_step": ms1 / K,
                          "note": "the same workload and steps on one GPU (all 26 fields, one sketch), measured by rank 0 in "
                                  "this run; value / (n_gpus * this) is the strong-scaling efficiency of the sharded run"}
            del one, ids1, g1
        barrier()
    line = None
    if rank == 0:
        peak, peak_kind = read_peaks()
        phases = {k: {"ms_per_step": v[0] / K, "launches_per_step": v[1] / K} for k, v in slots.items() if v[1] > 0}
        rank_ids = ids_per_step / world if wl.name != "weak26" else ids_per_step / world   # lookups this rank serves per step
        # share of distinct table rows among the lookups of the last timed batch (this rank's fields, global batch)
        u_rows = 1.0   # (weak26: every lookup counted with a row of its own)
        if wl.name != "weak26":
            last = wl.ids(W + K - 1, B)
            grp_ = run.grp if world == 1 else run.model.group
            own = last if world == 1 else last[run.model.plan.local_fields]
            u_rows = unique_row_share(grp_.row_codes(torch.from_numpy(np.ascontiguousarray(own)).to(dev)))
        # candidates for the dominant kernel: slots that time ONE kernel.  The two sort slots are sequences of four small
        # kernels per radix pass (12 to 17 launches per step); they are listed in `phases` and, kernel by kernel, in the
        # ncu launch list, where none of them comes near the streaming kernels.
        cand = {k: v for k, v in slots.items() if alg_bytes(k, DIM) > 0 and v[1] > 0 and k not in ("lookup_hash_sort", "row_sort")}
        # the sketch passes run in three modes (all buckets / later rounds / final pass) that are timed in slots of
        # their own: the kernel is ranked by their sum and reported on its all-bucket launches
        group = {"main_pass": ("main_pass", "main_pass_later_rounds", "main_pass_final"),
                 "lru_pass": ("lru_pass", "lru_pass_later_rounds")}
        weight = lambda k: sum(slots[g_][0] for g_ in group.get(k, (k,)) if g_ in slots)
        top = max(cand, key=weight) if cand else None
        roof = None
        if top:
            per_launch_ms = cand[top][0] / cand[top][1]
            # lookups one launch processes: the per-step kernels see every lookup of the step once; the
            # sketch passes run once or more per job over that job's window, and all windows of a step
            # add up to the step's lookups, so an average launch covers (lookups per step) / (launches per step)
            launches_per_step = cand[top][1] / K
            units = rank_ids / max(1.0, launches_per_step)
            ach = alg_bytes(top, DIM, u_rows) * units / (per_launch_ms / 1e3) / 1e9
            traffic = None
            tp = ROOT / "profiles" / "traffic.json"
            if tp.exists():
                try:
                    per_id = json.loads(tp.read_text()).get(top, {}).get("dram_bytes_per_id")
                    traffic = per_id * units if per_id else None
                except Exception:
                    traffic = None
            fused = FUSED_BYTES_PER_ID(DIM, u_rows) * ids_per_step / (ms / K / 1e3) / 1e9 / world
            main_roof = None
            if "main_pass" in slots and slots["main_pass"][1] > 0:
                mp_ms = slots["main_pass"][0] / slots["main_pass"][1]
                mp_units = rank_ids / max(1.0, slots["main_pass"][1] / K)
                mp_ach = alg_bytes("main_pass", DIM) * mp_units / (mp_ms / 1e3) / 1e9
                main_roof = {"achieved": mp_ach, "frac": mp_ach / peak, "ms_per_launch": mp_ms, "ids_per_launch": mp_units,
                             "note": "the all-bucket launches of the sketch's main pass (120 B per lookup)"}
            roof = {"bound": "hbm", "kernel": top, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                    "traffic": traffic, "peak_kind": peak_kind, "alg_bytes_per_id": alg_bytes(top, DIM, u_rows),
                    "distinct_rows_per_lookup": u_rows,
                    "ms_per_launch": per_launch_ms, "ids_per_launch": units, "main_pass": main_roof,
                    "fused_path": {"alg_bytes_per_id": FUSED_BYTES_PER_ID(DIM, u_rows), "achieved": fused, "frac": fused / peak,
                                   "frac_every_lookup_its_own_row": FUSED_BYTES_PER_ID(DIM, 1.0) * ids_per_step / (ms / K / 1e3) / 1e9 / world / peak,
                                   "note": "per GPU: whole-step algorithmic bytes / step time / n_gpus"}}
        dl = st1["lookups"] - st0["lookups"]
        mix = {"lookups": dl, "main_hit_frac": (st1["main_hits"] - st0["main_hits"]) / max(1, dl),
               "lru_visit_frac": (st1["lru_visits"] - st0["lru_visits"]) / max(1, dl),
               "rounds_per_step": (st1["rounds"] - st0["rounds"]) / K, "jobs_per_step": (st1["jobs"] - st0["jobs"]) / K,
               "refits_per_step": (st1["resets"] - st0["resets"]) / K, "seq_fallbacks": st1["seq_fallbacks"] - st0["seq_fallbacks"],
               "max_rounds": st1["max_rounds"], "note": "rank 0's sketch over the timed region of `value`"}
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": ms / K, "higher_is_better": True, "scaling": wl.scaling, "vs_baseline": None,
                "dtype": "f32", "data": "synthetic", "config": wl.config(B),
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": ms_e2e / K},
                "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "sketch_mix": mix, "phases": phases,
                "phases_note": "per-kernel CUDA-event times of a separate pass with the side-stream overlap switched off",
                "ms_per_step_profiled": ms_prof / K}
        if rank_info is not None:
            line["ranks"] = rank_info
        if single_ref is not None:
            line["single_gpu_same_workload"] = single_ref
        if world > 1:
            # bytes this rank stores into its peers per step and direction, against the time of the kernel that moves them
            R = 4 * DIM
            fg0 = len([f for f in range(wl.F) if f % world == 0])
            out_fwd = (world - 1) / world * B * fg0 * R
            out_bwd = (world - 1) / world * Bl * wl.F * R
            nv = {"peak_measured_GBs": 770.0, "peak_nominal_GBs": 900.0, "unit": "GB/s per direction per GPU (rank 0)"}
            if "embed_forward" in phases and phases["embed_forward"]["ms_per_step"] > 0:
                nv["gather_remote_store_GBs"] = out_fwd / (phases["embed_forward"]["ms_per_step"] / 1e3) / 1e9
            if "push_grads" in phases and phases["push_grads"]["ms_per_step"] > 0:
                nv["grad_push_GBs"] = out_bwd / (phases["push_grads"]["ms_per_step"] / 1e3) / 1e9
            nv["bytes_out_per_step"] = {"pooled_rows": out_fwd, "gradients": out_bwd}
            line["nvlink"] = nv
        if world == 1 and not args.no_dlrm:
            try:
                line["dlrm_samples_per_s"] = dlrm_figures()
            except Exception as e:   # informative only
                line["dlrm_samples_per_s"] = {"error": repr(e)}
        if world == 1 and not args.no_cpu_baseline:
            try:
                line["cpu_baseline"] = cpu_baseline_leg(args, wl)
            except Exception as e:  # the baseline is informative; never lose the GPU number to it
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "unavailable", "sample": repr(e)}
    if dist is not None and not args.no_dlrm:
        # Every rank takes part (the steps contain collectives).  The line above is complete without this figure: a
        # failure that every rank sees is reported in its place, and if the ranks stop answering each other a
        # watchdog lets rank 0 print the line as it stands and ends the process, so the step's numbers are never lost.
        import threading

        def give_up():
            if rank == 0:
                line["dlrm_samples_per_s"] = {"error": "no answer within 150 s; the figure was abandoned"}
                emit(line)
            os._exit(0)
        dog = threading.Timer(150.0, give_up)
        dog.daemon = True
        dog.start()
        try:
            fig = dlrm_figures_data_parallel()
        except Exception as e:
            fig = {"error": repr(e)}
        dist.barrier()   # (under the watchdog: a rank that failed alone would wait here for ranks that never come)
        dog.cancel()
        if rank == 0:
            line["dlrm_samples_per_s"] = fig
    if rank == 0:
        emit(line)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def dlrm_figures():
    """The metric's second figure on one GPU: samples/s of whole training steps (dense side on stock PyTorch, the
    CAFE embedding path from this library) at the three model configurations, on seeded synthetic data."""
    from cafe_b200 import dlrm_harness as H
    out = {}
    for name, argv in (("kaggle_dlrm_dim16_batch128", ["--data-set", "kaggle", "--mini-batch-size", "128", "--compress-rate", "0.001",
                                                        "--hash-rate", "0.3", "--nbatches", "150"]),
                       ("terabyte_dlrm_dim128_batch2048", ["--data-set", "terabyte", "--mini-batch-size", "2048", "--compress-rate",
                                                           "0.001", "--hash-rate", "0.3", "--nbatches", "60"]),
                       ("avazu_dcn_dim16_batch4096", ["--data-set", "avazu", "--model", "dcn", "--mini-batch-size", "4096",
                                                      "--compress-rate", "0.1", "--hash-rate", "0.7", "--nbatches", "60"])):
        r = H.run(H.make_parser().parse_args(["--sketch-flag", "--sketch-alpha", "1.0000005", "--warmup-batches", "20"] + argv))
        out[name] = {"samples_per_s": r["samples_per_s"], "ms_per_step": r["ms_per_step"], "sketch_fields": r["sketch_fields"],
                     "plain_fields": r["plain_fields"], "loss_last": r["loss_last"]}
        if "dcn" not in argv:
            # the same steps with the dot interaction through the library's kernels (not part of the figure above,
            # whose dense side is stock PyTorch throughout)
            r = H.run(H.make_parser().parse_args(["--sketch-flag", "--sketch-alpha", "1.0000005", "--warmup-batches", "20",
                                                  "--fused-interaction"] + argv))
            out[name]["with_fused_interaction"] = {"samples_per_s": r["samples_per_s"], "ms_per_step": r["ms_per_step"],
                                                   "loss_last": r["loss_last"]}
    out["note"] = ("whole training steps: stock-PyTorch MLPs / interaction / loss / SGD around the library's embedding path; "
                   "ids arrive as host tensors every step")
    return out


def dlrm_figures_data_parallel():
    """The same figure on several GPUs, weak scaling: every rank trains on its own batches of the single-GPU size, the
    embedding fields are sharded over the ranks (their owners serve the global batch), the dense side is replicated
    with its gradients summed every step (the Avazu shape's 13 small plain tables are part of that replicated side;
    its 9 sketch fields are sharded).  Called by every rank of the job; all return the whole job's samples/s."""
    from cafe_b200 import dlrm_harness as H
    out = {}
    for name, argv in (("kaggle_dlrm_dim16_batch128_per_gpu", ["--data-set", "kaggle", "--mini-batch-size", "128", "--compress-rate",
                                                                "0.001", "--hash-rate", "0.3", "--nbatches", "150"]),
                       ("terabyte_dlrm_dim128_batch2048_per_gpu", ["--data-set", "terabyte", "--mini-batch-size", "2048",
                                                                   "--compress-rate", "0.001", "--hash-rate", "0.3", "--nbatches", "60"]),
                       ("avazu_dcn_dim16_batch4096_per_gpu", ["--data-set", "avazu", "--model", "dcn", "--mini-batch-size", "4096",
                                                              "--compress-rate", "0.1", "--hash-rate", "0.7", "--nbatches", "60"])):
        r = H.run_data_parallel(H.make_parser().parse_args(["--sketch-flag", "--sketch-alpha", "1.0000005", "--warmup-batches", "20"]
                                                           + argv))
        out[name] = {k: r[k] for k in ("samples_per_s", "ms_per_step", "ranks", "global_batch", "sketch_fields", "plain_fields",
                                       "loss_last", "replicas_in_step")}
    out["note"] = ("whole training steps, weak scaling: fields sharded over the GPUs (lookup, insert, migration and SGD of the "
                   "global batch on the owners), stock-PyTorch MLPs / interaction / loss / SGD replicated, dense gradients "
                   "summed by one all-reduce per step; ids arrive as host tensors every step")
    return out


_RESULT_OUT = None


def keep_stdout_for_the_result():
    """Libraries loaded later write banners to file descriptor 1 (NCCL prints its version there at start-up).  The
    descriptor is kept aside for the JSON line and everything else that would go to it is sent to stderr."""
    global _RESULT_OUT
    if _RESULT_OUT is None:
        sys.stdout.flush()
        _RESULT_OUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(line: dict):
    out = _RESULT_OUT if _RESULT_OUT is not None else sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    keep_stdout_for_the_result()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto", choices=["auto", "micro", "cfg3", "weak26"])
    ap.add_argument("--drift-stride", type=int, default=100, help="cfg3: workload steps per bench step")
    ap.add_argument("--batch", type=int, default=BATCH, help="global batch (samples per step)")
    ap.add_argument("--cpu-batch", type=int, default=BATCH, help="batch of the CPU reference path")
    ap.add_argument("--cpu-steps", type=int, default=3, help="timed steps of the cpu_baseline leg of our arm")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-dlrm", action="store_true", help="skip the DLRM / DCN samples-per-second figures")
    ap.add_argument("--no-single-ref", action="store_true", help="cfg3 on several GPUs: skip the one-GPU run of the same workload")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="multi-GPU exchange of pooled rows / gradients")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.warmup < 3:
        args.warmup = 3
    if args.workload == "auto":
        args.workload = "micro" if world == 1 else "cfg3"
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
