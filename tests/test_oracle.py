"""The CPU oracle (C restatement) against the reference's golden vectors.

Fixtures under tests/golden/ were produced by the compiled reference (make_golden.py).  Where the
reference checkout is present the compiled reference is also driven live and compared state for state.
"""
import json
from pathlib import Path

import numpy as np
import pytest

from kat_stream import KATS, SplitMix64, kat_call, run_kat
from oracle.hotsketch import OracleSketch, ReferenceSketch, ref_available, states_equal

GOLDEN = Path(__file__).resolve().parent / "golden"
STATE_KEYS = ["main_val", "main_cnt", "main_dic", "main_flip", "lru_val", "lru_cnt", "lru_dic", "lru_t",
              "lru_flip", "queue"]


def _digest(st):
    import hashlib
    h = hashlib.sha256()
    for k in STATE_KEYS:
        h.update(np.ascontiguousarray(st[k]).tobytes())
    h.update(json.dumps([st["thr_bits"], st["real_n"], st["num"], st["t"], st["gflip"]]).encode())
    return h.hexdigest()


@pytest.mark.parametrize("idx", range(len(KATS)))
def test_known_answer_hashes(idx):
    want = json.loads((GOLDEN / "kat_hashes.json").read_text())[idx]
    k = KATS[idx]
    s = OracleSketch(k["lim"], k["thr"], 1, k["alpha"])
    fnv, newhot, hotq = run_kat(s, k["calls"], k["n"], k["dom"])
    assert (fnv, newhot, hotq) == (want["fnv1a64"], want["newhot"], want["hotq"])
    st = s.state()
    assert _digest(st) == want["state_sha256"]
    assert len(st["queue"]) == want["queue_len"]


def test_small_stream_outputs_and_state():
    g = np.load(GOLDEN / "small_stream.npz")
    s = OracleSketch(int(g["lim"]), float(g["thr"]), 1, float(g["alpha"]))
    for c in range(g["ids"].shape[0]):
        assert np.array_equal(s.batch_query(g["ids"][c]), g["q0"][c])
        assert np.array_equal(s.batch_insert_val(g["ids"][c], g["v"][c]), g["mask"][c])
        assert np.array_equal(s.batch_query(g["ids"][c]), g["q1"][c])
    st = s.state()
    for k in STATE_KEYS:
        a, b = st[k], g[k]
        if a.dtype == np.float32:
            a, b = a.view(np.uint32), b.view(np.uint32)
        assert np.array_equal(a, b), k
    assert [st["thr_bits"], st["real_n"], st["num"], st["t"], st["gflip"]] == list(g["scalars"])
    c = s.counters()
    # the stream is meant to reach every path of the algorithm
    assert c["resets"] >= 3 and c["flips"] >= 1 and c["promote_own"] > 0 and c["promote_victim"] > 0
    assert c["insert_fail"] > 0 and c["lru_hit"] > 0


@pytest.mark.skipif(not ref_available(), reason="reference checkout absent")
@pytest.mark.parametrize("lim,thr,alpha,calls,n,dom,unit", [
    (64, 1, 1.5, 60, 32, 400, False),
    (500, 3, 1.05, 300, 50, 20000, False),
    (2000, 1, 1.0000005, 50, 1000, 100000, False),
    (300, 1, 1.2, 100, 64, 2500, True),      # batch_insert (unit counts)
    (1000, 500, 1.0000005, 40, 500, 3000, False),  # high threshold, no resets
])
def test_live_reference_state_for_state(lim, thr, alpha, calls, n, dom, unit):
    a, b = ReferenceSketch(lim, thr, 1, alpha), OracleSketch(lim, thr, 1, alpha)
    rng = SplitMix64(lim * 31 + n)
    for c in range(calls):
        ids, v = kat_call(rng, n, dom)
        if c % 7 == 3:
            ids[::5] = 0  # id 0 doubles as the empty-slot marker in the reference; must match too
        assert np.array_equal(a.batch_query(ids), b.batch_query(ids))
        if unit:
            assert np.array_equal(a.batch_insert(ids), b.batch_insert(ids))
        else:
            assert np.array_equal(a.batch_insert_val(ids, v), b.batch_insert_val(ids, v))
        assert a.analyse(ids) == b.analyse(ids) and a.analyse1(ids) == b.analyse1(ids)
        if c % 10 == 9 or c == calls - 1:
            assert states_equal(a.state(), b.state()) == [], f"call {c}"


def test_empty_call_is_a_call():
    """A zero-length insert still advances the decay clock (the reference multiplies per call)."""
    s = OracleSketch(100, 1, 1, 1.5)
    e = np.zeros(0, np.uint32)
    assert s.batch_insert_val(e, np.zeros(0, np.float32)).size == 0
    assert s.state()["batch_num"] == 1 and s.state()["decay_importance"] == 1.5
    assert s.batch_query(e).size == 0
