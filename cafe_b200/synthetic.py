"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

Stand-ins for the public click-log datasets the reference trains on (their files are not available):
per field, a rank is drawn from a bounded Zipf(s) law by inverting the CDF of its continuous
approximation, and mapped to an id by a seeded bijection of [0, n) (a cycle-walking Feistel network,
so that 40M-id fields need no permutation table).  Everything is generated on the host with numpy
from (seed, step, field), so the CPU baseline and the GPU path can be fed identical arrays.
"""
from __future__ import annotations

import numpy as np

KAGGLE_CARDS = [1460, 583, 10131227, 2202608, 305, 24, 12517, 633, 3, 93145, 5683, 8351593, 3194, 27, 14992, 5461306,
                10, 5652, 2173, 4, 7046547, 18, 15, 286181, 105, 142572]
TERABYTE_CARDS = [39884406, 39043, 17289, 7420, 20263, 3, 7120, 1543, 63, 38532951, 2953546, 403346, 10, 2208, 11938,
                  155, 4, 976, 14, 39979771, 25641295, 39664984, 585935, 12972, 108, 36]
AVAZU_CARDS = [7, 7, 4737, 7745, 26, 8552, 559, 36, 2686408, 6729486, 8251, 5, 4, 2626, 8, 9, 435, 4, 68, 172, 60, 16]
MICRO_CARDS = [40_000_000] * 26


def _mix(x: np.ndarray, key: int) -> np.ndarray:
    """32-bit avalanche hash of x with a round key (uint64 arithmetic, values < 2**32)."""
    x = (x ^ np.uint64(key & 0xFFFFFFFF)) & np.uint64(0xFFFFFFFF)
    x = (x * np.uint64(0x9E3779B1)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(15)
    x = (x * np.uint64(0x85EBCA77)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(13)
    x = (x * np.uint64(0xC2B2AE3D)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(16)
    return x


def feistel_permute(r: np.ndarray, n: int, seed: int) -> np.ndarray:
    """A bijection of [0, n): 4-round Feistel network on the next even power of two, re-applied to
    values that land outside [0, n) (cycle walking)."""
    if n <= 1:
        return np.zeros_like(r, dtype=np.int64)
    bits = max(2, int(n - 1).bit_length())
    bits += bits & 1
    half = bits // 2
    mask = np.uint64((1 << half) - 1)
    x = r.astype(np.uint64)
    todo = np.ones(x.shape, bool)
    while todo.any():
        v = x[todo]
        left, right = v >> np.uint64(half), v & mask
        for rnd in range(4):
            left, right = right, left ^ (_mix(right, seed * 4 + rnd + 1) & mask)
        v = (left << np.uint64(half)) | right
        x[todo] = v
        todo[todo] = v >= np.uint64(n)
    return x.astype(np.int64)


def zipf_ranks(u: np.ndarray, n: int, s: float) -> np.ndarray:
    """Bounded Zipf(s) ranks in [0, n) from uniforms in [0, 1)."""
    if abs(s - 1.0) < 1e-9:
        r = np.floor(np.power(n + 1.0, u)) - 1
    else:
        a = 1.0 - s
        r = np.floor(np.power(u * (np.power(n + 1.0, a) - 1.0) + 1.0, 1.0 / a)) - 1
    return np.clip(r, 0, n - 1).astype(np.int64)


def batch_ids(cards, batch: int, s: float, seed: int, step: int, dtype=np.int64) -> np.ndarray:
    """ids [F, batch]: field f's ids are Zipf(s) over [0, cards[f]) through field f's permutation."""
    out = np.empty((len(cards), batch), dtype)
    for f, n in enumerate(cards):
        rng = np.random.Generator(np.random.Philox(key=[seed, 0], counter=[0, 0, step, f]))
        u = rng.random(batch)
        out[f] = feistel_permute(zipf_ranks(u, int(n), s), int(n), seed * 1000 + f).astype(dtype)
    return out


def drift_exponent(step: int, s0: float = 1.05, s1: float = 1.2, horizon: int = 10_000) -> float:
    """Zipf exponent of the drifting workload: linear from s0 at step 0 to s1 at `horizon`, constant afterwards."""
    return s0 + (s1 - s0) * min(max(step, 0), horizon) / float(horizon)


def drift_remap(ids: np.ndarray, n: int, seed: int, field: int, epochs: int, den: int = 20) -> np.ndarray:
    """The re-permutations of the drifting workload applied to ids of one field.

    Epoch j (j = 1..epochs) re-permutes, among themselves, the ids whose remainder modulo `den` equals a
    seeded residue c_j: 1/den of the id space (5 % for den = 20) moves, everything else stays.  Each epoch
    is a bijection of [0, n) (a Feistel permutation of the quotients within one residue class), so the
    composition is one too and no table is needed for 40M-id fields."""
    x = ids.astype(np.int64, copy=True)
    if n < 2 * den:
        return x
    for j in range(1, epochs + 1):
        c = int(_mix(np.array([j], np.uint64), seed * 7919 + field * 131 + 17)[0] % np.uint64(den))
        cnt = (n - c + den - 1) // den            # ids in [0, n) with id % den == c
        sel = (x % den) == c
        if cnt > 1 and sel.any():
            x[sel] = feistel_permute(x[sel] // den, int(cnt), seed * 1000 + field * 37 + 5000 + j) * den + c
    return x


def drift_batch_ids(cards, batch: int, seed: int, step: int, s0: float = 1.05, s1: float = 1.2, horizon: int = 10_000,
                    period: int = 1000, den: int = 20, dtype=np.int64) -> np.ndarray:
    """ids [F, batch] of the drifting Terabyte-shaped workload: the Zipf exponent moves from s0 to s1 over
    `horizon` steps and, every `period` steps, 1/den of every field's ids are re-permuted (drift_remap), so
    that ids leave and enter the hot set while training runs."""
    s = drift_exponent(step, s0, s1, horizon)
    out = np.empty((len(cards), batch), dtype)
    for f, n in enumerate(cards):
        rng = np.random.Generator(np.random.Philox(key=[seed, 0], counter=[0, 0, step, f]))
        u = rng.random(batch)
        base = feistel_permute(zipf_ranks(u, int(n), s), int(n), seed * 1000 + f)
        out[f] = drift_remap(base, int(n), seed, f, step // period, den).astype(dtype)
    return out


def dense_features(batch: int, seed: int, step: int, num: int = 13) -> np.ndarray:
    """log(1 + round(Exp(mean 20))) as fp32, the dense side of the Criteo-shaped configurations."""
    rng = np.random.Generator(np.random.Philox(key=[seed, 1], counter=[0, 0, step, 0]))
    return np.log1p(np.rint(rng.exponential(20.0, size=(batch, num)))).astype(np.float32)


def labels(batch: int, p: float, seed: int, step: int) -> np.ndarray:
    rng = np.random.Generator(np.random.Philox(key=[seed, 2], counter=[0, 0, step, 0]))
    return (rng.random(batch) < p).astype(np.float32)


def gradients(batch: int, fields: int, dim: int, seed: int, step: int, std: float = 0.01) -> np.ndarray:
    """Stand-in for dL/d(pooled embedding): N(0, std^2) fp32 [batch, fields, dim]."""
    rng = np.random.Generator(np.random.Philox(key=[seed, 3], counter=[0, 0, step, 0]))
    return (rng.standard_normal((batch, fields, dim), dtype=np.float32) * np.float32(std)).astype(np.float32)
