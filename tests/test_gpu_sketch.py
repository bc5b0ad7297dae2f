"""Bit-exact parity of the CUDA HotSketch with the sequential CPU oracle, through the C ABI.

Every case feeds identical (id, importance) arrays to both sides and compares per-lookup results
(query, insert mask, post-insert row) and the complete state (both bucket tables, the free-row FIFO
in order, threshold, counters, LRU clock)."""
import json
from pathlib import Path

import numpy as np
import pytest

from kat_stream import KATS, run_kat
from sketch_driver import drive as _drive

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


class GpuSketch:
    """Adapter giving cafe_b200.HotSketch the interface the shared driver expects."""

    def __init__(self, lim, thr, adjust, alpha, cap, parallel=True):
        import cafe_b200
        self.sk = cafe_b200.HotSketch(lim, thr, adjust, alpha, max_lookups=cap)
        self.mode = cafe_b200.INSERT_PARALLEL if parallel else cafe_b200.INSERT_SEQUENTIAL
        self.last_rc = 0
        self.last_post_row = None

    def batch_query(self, ids):
        return self.sk.batch_query(ids)

    def insert_segments(self, ids, v, seg_off):
        import torch
        t = torch.from_numpy(np.ascontiguousarray(np.asarray(ids).astype(np.uint32)).view(np.int32)).cuda()
        vi = None if v is None else torch.from_numpy(np.ascontiguousarray(v, np.float32)).cuda()
        mask, post = self.sk.insert(t, vi, list(seg_off), self.mode)
        self.last_rc = self.sk.last_status
        self.last_post_row = post.cpu().numpy()
        return mask.cpu().numpy()

    def batch_insert_val(self, ids, v=None):
        return self.insert_segments(ids, v, [0, len(ids)])

    def set_window(self, w):
        self.sk.tune(window=w)

    def set_round_cap(self, c):
        self.sk.tune(round_cap=c)

    def state(self):
        return self.sk.state()

    def stats(self):
        return self.sk.stats()


def drive(*a, **k):
    return _drive(lambda lim, thr, adj, alpha, cap, par: GpuSketch(lim, thr, adj, alpha, cap, par), *a, **k)


def test_sequential_kernel():
    st = drive(200, 1, 1.3, 40, 96, 3000, 1, parallel=False)
    assert st["resets"] >= 3 and st["flips"] == 1


@pytest.mark.parametrize("fuse", [1, 4, 13])
def test_small_sketch_all_paths(fuse):
    st = drive(200, 1, 1.3, 52, 96, 3000, fuse)
    assert st["resets"] >= 3 and st["flips"] >= 1 and st["events"] > 0 and st["seq_fallbacks"] == 0


def test_fused_fields_with_refits_cutting_jobs():
    st = drive(20000, 1, 1.0000005, 52, 4096, 5000000, 26)
    assert st["truncated_jobs"] > 0 and st["resets"] > 0 and st["seq_fallbacks"] == 0


def test_kaggle_sized_sketch_fused_26():
    drive(13505, 1, 1.0000005, 260, 128, 33762577, 26)


def test_threshold_above_one_and_decay():
    st = drive(1000, 2, 1.01, 1200, 64, 200000, 8)
    assert st["flips"] >= 1


def test_unit_counts_zero_ids_ragged():
    drive(300, 1, 1.2, 60, 64, 2500, 3, unit=True)
    drive(300, 1, 1.2, 60, 64, 2500, 3, zero_ids=True)
    drive(200, 1, 1.3, 60, 50, 3000, 6, ragged=True)


def test_heavy_duplicates():
    drive(100, 1, 1.1, 30, 600, 40, 3)


def test_small_sketch_large_calls():
    """Hundreds of lookups per bucket and call (the LRU pass then replays compacted miss lists, every main bucket is
    fed by a warp, and long stretches of one hot id are remembered between rounds)."""
    st = drive(60, 1, 1.2, 24, 2000, 300, 2)
    assert st["resets"] > 0 and st["seq_fallbacks"] == 0
    drive(400, 2, 1.0000005, 12, 40000, 3000, 3, seed=11)
    drive(300, 1, 1.0000005, 8, 60000, 40, 2, seed=12)      # a 40-id domain: stretches of thousands of lookups of one id


def test_few_lru_buckets_thousands_of_misses_each():
    """Thresholds above 1 and sketches of a few dozen to a few hundred slots fed tens of thousands of lookups per call:
    every LRU bucket sees hundreds to thousands of main-table misses per call, which the warps replay a chunk of 32
    at a time (hits, misses, replaced entries that come back, empty slots, ids equal to 0, unit and random counts)."""
    drive(100, 3, 1.0000005, 10, 30000, 2000, 2, seed=21)
    drive(60, 2, 1.2, 12, 20000, 500, 3, seed=22, unit=True)
    drive(358, 1, 1.0000005, 12, 65536, 300000, 6, seed=23)     # a shard of small fields: 6 fields x 65536 on 358 slots
    drive(100, 3, 1.1, 6, 30000, 2000, 2, seed=24, zero_ids=True)
    drive(40, 4, 1.0000005, 8, 5000, 60, 2, seed=25)            # a 60-id domain on 4 LRU buckets: mostly hits
    drive(2000, 2, 1.0000005, 6, 65536, 5000000, 3, seed=26)


def test_round_cap_fallback_is_exact():
    st = drive(200, 1, 1.3, 40, 96, 3000, 4, round_cap=2)
    assert st["seq_fallbacks"] > 0


def test_large_batch_microbenchmark_shape():
    """65536-id calls on a sketch of the microbenchmark's size (lim 665600), 4 fields fused."""
    st = drive(665600, 1, 1.0000005, 8, 65536, 40_000_000, 4)
    assert st["seq_fallbacks"] == 0


@pytest.mark.parametrize("idx", [0, 2])
def test_known_answer_hashes_through_gpu(idx):
    want = json.loads((GOLDEN / "kat_hashes.json").read_text())[idx]
    k = KATS[idx]
    s = GpuSketch(k["lim"], k["thr"], 1, k["alpha"], k["n"])
    fnv, newhot, hotq = run_kat(s, k["calls"], k["n"], k["dom"])
    assert (fnv, newhot, hotq) == (want["fnv1a64"], want["newhot"], want["hotq"])


def test_golden_small_stream_from_reference():
    g = np.load(GOLDEN / "small_stream.npz")
    s = GpuSketch(int(g["lim"]), float(g["thr"]), 1, float(g["alpha"]), g["ids"].shape[1])
    for c in range(g["ids"].shape[0]):
        assert np.array_equal(s.batch_query(g["ids"][c]), g["q0"][c])
        assert np.array_equal(s.batch_insert_val(g["ids"][c], g["v"][c]), g["mask"][c])
        assert np.array_equal(s.batch_query(g["ids"][c]), g["q1"][c])
    st = s.state()
    for k in ["main_val", "main_cnt", "main_dic", "main_flip", "lru_val", "lru_cnt", "lru_dic", "lru_t", "lru_flip", "queue"]:
        a, b = st[k], g[k]
        if a.dtype == np.float32:
            a, b = a.view(np.uint32), b.view(np.uint32)
        assert np.array_equal(a, b), k
    assert [st["thr_bits"], st["real_n"], st["num"], st["t"], st["gflip"]] == list(g["scalars"])


def test_state_save_and_restore():
    import cafe_b200
    a = GpuSketch(300, 1, 1, 1.2, 64 * 3)
    drive_ids = np.random.default_rng(0).integers(1, 2500, size=(10, 192)).astype(np.uint32)
    v = np.random.default_rng(1).random((10, 192)).astype(np.float32) * 3
    for c in range(5):
        a.batch_insert_val(drive_ids[c], v[c])
    st = a.state()
    b = cafe_b200.HotSketch(300, 1, 1, 1.2, max_lookups=192)
    b.load_state(st)
    for c in range(5, 10):
        ma = a.batch_insert_val(drive_ids[c], v[c])
        mb = b.batch_insert_val(drive_ids[c], v[c])
        assert np.array_equal(ma, mb)
    from oracle.hotsketch import states_equal
    assert states_equal(a.state(), b.state()) == []


def test_reference_ctypes_abi_host_pointers():
    """The six symbols of the reference's sklib.so, called the way its Python calls them."""
    import ctypes
    import cafe_b200
    from oracle.hotsketch import OracleSketch
    lib = cafe_b200.load_library()
    lib.init(500, 2, 1, 1.05)
    o = OracleSketch(500, 2, 1, 1.05)
    rng = np.random.default_rng(3)
    for c in range(30):
        ids = rng.integers(1, 4000, size=100).astype(np.uint32)
        v = (rng.random(100) * 4).astype(np.float32)
        ip = ids.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32))
        q = np.ctypeslib.as_array(lib.batch_query(ip, 100), shape=(100,)).copy()
        assert np.array_equal(q, o.batch_query(ids))
        if c % 2:
            m = np.ctypeslib.as_array(lib.batch_insert_val(ip, v.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), 100), shape=(100,)).copy()
            assert np.array_equal(m, o.batch_insert_val(ids, v))
        else:
            m = np.ctypeslib.as_array(lib.batch_insert(ip, 100), shape=(100,)).copy()
            assert np.array_equal(m, o.batch_insert(ids))
        assert lib.analyse(ip, 100) == o.analyse(ids) and lib.analyse1(ip, 100) == o.analyse1(ids)


@pytest.mark.parametrize("block", range(4))
def test_random_configurations(block):
    """Seeded random shapes: small to mid-size sketches, calls of 200-6000 ids over domains from 30 ids (long
    buckets whose ids alternate) to 200 000, fused windows, ragged and empty calls, id 0, unit counts.
    Masks, post-insert rows and the whole state must equal the sequential algorithm's after every job."""
    for seed in range(block * 12, block * 12 + 12):
        r = np.random.default_rng(seed)
        lim = int(r.integers(40, 3000)); thr = int(r.integers(1, 5)); alpha = float(r.choice([1.0000005, 1.05, 1.5]))
        n = int(r.integers(200, 6000)); dom = int(r.choice([30, 200, 3000, 200000])); fuse = int(r.integers(1, 8))
        drive(lim, thr, alpha, fuse * 6, n, dom, fuse, seed=1000 + seed, zero_ids=seed % 3 == 0, ragged=seed % 4 == 1,
              unit=seed % 5 == 2)
