"""Seeded known-answer stream shared by the golden-vector generator and the tests.

splitmix64 (state 42) drives, per element and in this order, an id and an importance:
    u  = (next() >> 11) * 2**-53 ; w = u*u ; w = w*w ; id = 1 + uint32(w * (dom - 1))
    v  = float32((next() % 1024) + 1) / 256
Per call the stream yields N fresh elements.  Outputs of a run are folded into FNV-1a-64 over the
little-endian bytes of every int32 result, in the order query / insert / query per call.
"""
from __future__ import annotations

import numpy as np

_M64 = (1 << 64) - 1
FNV_OFFSET = 1469598103934665603
FNV_PRIME = 1099511628211


class SplitMix64:
    def __init__(self, seed: int = 42):
        self.s = seed & _M64

    def take(self, n: int) -> np.ndarray:
        """Next n outputs as uint64 (vectorised: the state advances by a constant per draw)."""
        with np.errstate(over="ignore"):
            k = np.arange(1, n + 1, dtype=np.uint64)
            z = np.uint64(self.s) + k * np.uint64(0x9E3779B97F4A7C15)
            self.s = int(z[-1]) if n else self.s
            z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
            z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
            return z ^ (z >> np.uint64(31))


def kat_call(rng: SplitMix64, n: int, dom: int):
    r = rng.take(2 * n)
    u = (r[0::2] >> np.uint64(11)).astype(np.float64) * (2.0 ** -53)
    w = u * u
    w = w * w
    ids = (1 + (w * (dom - 1)).astype(np.uint32)).astype(np.uint32)
    v = ((r[1::2] % np.uint64(1024)) + np.uint64(1)).astype(np.float32) / np.float32(256.0)
    return ids, v.astype(np.float32)


def fnv1a64(h: int, arr: np.ndarray) -> int:
    for b in np.ascontiguousarray(arr, dtype="<i4").tobytes():
        h = ((h ^ b) * FNV_PRIME) & _M64
    return h


def run_kat(sketch, calls: int, n: int, dom: int, seed: int = 42):
    """Drive query / insert_val / query for `calls` calls; returns (fnv hex, newhot, hotq)."""
    rng = SplitMix64(seed)
    h = FNV_OFFSET
    newhot = hotq = 0
    chunks = []
    for _ in range(calls):
        ids, v = kat_call(rng, n, dom)
        q0 = sketch.batch_query(ids)
        m = sketch.batch_insert_val(ids, v)
        q1 = sketch.batch_query(ids)
        chunks += [q0, m, q1]
        newhot += int(m.sum())
        hotq += int((q1 < 0).sum())
    # hashing byte-by-byte in Python is slow; fold the concatenation with a small C-speed loop
    h = _fnv_fast(h, np.concatenate(chunks))
    return f"{h:016x}", newhot, hotq


def _fnv_fast(h: int, arr: np.ndarray) -> int:
    data = np.ascontiguousarray(arr, dtype="<i4").tobytes()
    # process in Python ints but with local variable binding; ~10 MB/s is enough for the KAT sizes
    prime, mask = FNV_PRIME, _M64
    for b in data:
        h = ((h ^ b) * prime) & mask
    return h


KATS = [
    dict(lim=1000, thr=2, alpha=1.01, calls=2000, n=64, dom=200000),
    dict(lim=20000, thr=1, alpha=1.0000005, calls=300, n=4096, dom=5000000),
    dict(lim=13505, thr=1, alpha=1.0000005, calls=2600, n=128, dom=33762577),
]
