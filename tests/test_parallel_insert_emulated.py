"""Exactness of the parallel (round-based) insert, checked on the CPU.

The CUDA kernels call per-bucket / per-position functions from cafe_b200/csrc/sketch_core.cuh under
the driver of sketch_engine.h.  tests/hostemu compiles the same two headers with a loop-based
backend; here that build is compared, state for state and output for output, with the sequential
oracle on seeded streams that reach every path (promotions of both kinds, failed promotions that
push a row back, flip-bit decay, threshold re-fits at call boundaries inside a fused job).
"""
import numpy as np
import pytest

from hostemu import EmuSketch
from sketch_driver import drive as _drive


def drive(*a, **k):
    return _drive(lambda lim, thr, adj, alpha, cap, par: EmuSketch(lim, thr, adj, alpha, cap=cap, parallel=par), *a, **k)


def test_sequential_kernel_logic_matches_oracle():
    st = drive(200, 1, 1.3, 40, 96, 3000, 1, parallel=False)
    assert st["resets"] >= 3 and st["flips"] == 1


@pytest.mark.parametrize("fuse", [1, 4, 13])
def test_small_sketch_all_paths(fuse):
    st = drive(200, 1, 1.3, 52, 96, 3000, fuse)
    assert st["resets"] >= 3 and st["flips"] >= 1 and st["events"] > 0 and st["seq_fallbacks"] == 0


def test_fused_fields_with_refits_cutting_jobs():
    st = drive(20000, 1, 1.0000005, 52, 4096, 5000000, 26)
    assert st["truncated_jobs"] > 0 and st["resets"] > 0 and st["seq_fallbacks"] == 0


def test_many_shortened_jobs_replay_only_what_the_cut_touched():
    """Jobs sized without the crossing-rate prediction: a threshold re-fit falls due inside most of them, the job is
    shortened to the boundary before it, and only the buckets that the dropped lookups touched replay (several shapes,
    random and unit counts)."""
    st = drive(2000, 1, 1.0000005, 52, 1024, 200000, 26, seed=31, size_jobs_by_rate=False)
    assert st["truncated_jobs"] >= 5 and st["seq_fallbacks"] == 0
    st = drive(500, 1, 1.05, 48, 600, 20000, 12, seed=32, size_jobs_by_rate=False)
    assert st["truncated_jobs"] >= 5 and st["seq_fallbacks"] == 0
    st = drive(3000, 1, 1.0000005, 78, 2048, 2000000, 26, seed=34, size_jobs_by_rate=False, unit=True)
    assert st["truncated_jobs"] >= 5 and st["seq_fallbacks"] == 0
    st = drive(200, 1, 1.3, 52, 96, 3000, 13, seed=36, size_jobs_by_rate=False)
    assert st["truncated_jobs"] >= 3 and st["seq_fallbacks"] == 0


def test_kaggle_sized_sketch_fused_26():
    st = drive(13505, 1, 1.0000005, 260, 128, 33762577, 26)
    assert st["seq_fallbacks"] == 0


def test_threshold_above_one_and_decay():
    st = drive(1000, 2, 1.01, 1200, 64, 200000, 8)
    assert st["flips"] >= 1 and st["seq_fallbacks"] == 0


def test_high_threshold_no_refit():
    drive(1000, 500, 1.0000005, 40, 500, 3000, 4)


def test_unit_counts_batch_insert():
    drive(300, 1, 1.2, 60, 64, 2500, 3, unit=True)


def test_id_zero_is_reproduced():
    # id 0 doubles as the empty-slot marker in the reference (sketch.cpp:238); same quirks expected
    drive(300, 1, 1.2, 60, 64, 2500, 3, zero_ids=True)


def test_ragged_and_empty_segments():
    drive(200, 1, 1.3, 60, 50, 3000, 6, ragged=True)


def test_heavy_duplicates_tiny_domain():
    # a handful of ids repeated hundreds of times per call: long same-bucket runs, in batch order
    drive(100, 1, 1.1, 30, 600, 40, 3)


def test_round_cap_falls_back_to_sequential_and_stays_exact():
    st = drive(200, 1, 1.3, 40, 96, 3000, 4, round_cap=2)
    assert st["seq_fallbacks"] > 0


@pytest.mark.parametrize("seed", range(6))
def test_random_shapes(seed):
    r = np.random.default_rng(seed)
    lim = int(r.integers(40, 400))
    thr = int(r.integers(1, 4))
    alpha = float(r.choice([1.0000005, 1.05, 1.5]))
    n = int(r.integers(1, 200))
    dom = int(r.integers(20, 5000))
    fuse = int(r.integers(1, 9))
    drive(lim, thr, alpha, fuse * 8, n, dom, fuse, seed=100 + seed)


@pytest.mark.parametrize("block", range(4))
def test_random_configurations(block):
    """Seeded random shapes on the emulated backend: sketches of 25 to 13 733 slots, calls of 50 to 12 000 ids over
    domains of 12 ids (a few long buckets whose ids alternate) to 5 000 000, 1 to 26 calls fused, thresholds 1-4,
    slow and fast decay, ragged and empty calls, id 0, unit counts; every other case sizes its jobs without the
    crossing-rate prediction, so that re-fits fall due inside jobs and shorten them."""
    for seed in range(block * 40, block * 40 + 40):
        r = np.random.default_rng(seed)
        lim = int(r.choice([25, 40, 100, 300, 1000, 3000, 13733]))
        thr = int(r.integers(1, 5)); alpha = float(r.choice([1.0000005, 1.05, 1.5]))
        n = int(r.choice([50, 200, 1000, 4000, 12000])); dom = int(r.choice([12, 30, 200, 3000, 200000, 5000000]))
        fuse = int(r.integers(1, 27))
        kw = dict(seed=5000 + seed, zero_ids=seed % 3 == 0, ragged=seed % 4 == 1, unit=seed % 5 == 2)
        if seed % 2:
            kw["size_jobs_by_rate"] = False
        drive(lim, thr, alpha, fuse * int(r.integers(2, 6)), n, dom, fuse, **kw)
