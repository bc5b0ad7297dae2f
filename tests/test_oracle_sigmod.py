"""The CPU oracle of the one-stage HotSketch (oracle/sigmod_oracle.c) against the reference.

tests/golden/sigmod_stream.npz was produced by the reference's own ArtifactEvaluation/embeddings/sketch.cpp
(make_golden_sigmod.py); where the reference checkout is present the compiled reference is also driven live."""
from pathlib import Path

import numpy as np
import pytest

from oracle.sigmod import OracleSigmod, ReferenceSigmod, ref_available

GOLDEN = Path(__file__).resolve().parent / "golden" / "sigmod_stream.npz"


def same_state(a, b):
    bad = [k for k in ("val", "dic", "queue") if not np.array_equal(a[k], b[k])]
    if not np.array_equal(a["cnt"].view(np.uint32), b["cnt"].view(np.uint32)):
        bad.append("cnt")
    if a["num"] != b["num"] or a["tot"] != b["tot"]:
        bad.append("scalars")
    return bad


def replay_golden(make):
    g = np.load(GOLDEN)
    s = make(int(g["lim"]), int(g["k"]), float(g["dr"]))
    for c in range(g["ids"].shape[0]):
        assert np.array_equal(s.batch_query(g["ids"][c]), g["q0"][c]), f"call {c}: query before"
        m = s.batch_insert_val(g["ids"][c], g["v"][c]) if c % 3 else s.batch_insert(g["ids"][c])
        assert np.array_equal(m, g["mask"][c]), f"call {c}: insert result"
        assert np.array_equal(s.batch_query(g["ids"][c]), g["q1"][c]), f"call {c}: query after"
    st = s.state()
    want = dict(val=g["val"], cnt=g["cnt"], dic=g["dic"], queue=g["queue"], num=int(g["num"]), tot=float(g["tot"]))
    assert same_state(st, want) == []
    return st


def test_restatement_reproduces_the_reference_fixture():
    st = replay_golden(OracleSigmod)
    assert st["num"] > 299          # rows were handed out again after decays freed them


@pytest.mark.skipif(not ref_available(), reason="reference checkout absent")
@pytest.mark.parametrize("lim,k,dr,calls,n,dom,zipf", [(50, 3, 0.8, 80, 200, 900, 1.3), (2000, 20, 0.99, 40, 4096, 100000, 1.1),
                                                       (128, 1, 0.5, 60, 333, 5000, 1.5)])
def test_live_reference_state_for_state(lim, k, dr, calls, n, dom, zipf):
    rng = np.random.default_rng(lim + k)
    o, r = OracleSigmod(lim, k, dr), ReferenceSigmod(lim, k, dr)
    for c in range(calls):
        ids = np.minimum(rng.zipf(zipf, size=n), dom).astype(np.uint32)
        v = (rng.integers(1, 2048, size=n) / 256.0).astype(np.float32)
        assert np.array_equal(o.batch_query(ids), r.batch_query(ids))
        if c % 4 == 3:
            assert np.array_equal(o.batch_insert(ids), r.batch_insert(ids))
        else:
            assert np.array_equal(o.batch_insert_val(ids, v), r.batch_insert_val(ids, v))
        assert same_state(o.state(), r.state()) == [], f"call {c}"


def test_update_rebuilds_the_free_row_list():
    o = OracleSigmod(100, 2, 0.9)
    rng = np.random.default_rng(1)
    for _ in range(10):
        o.batch_insert(np.minimum(rng.zipf(1.4, size=300), 2000).astype(np.uint32))
    st = o.state()
    held = set(st["dic"][st["dic"] != 0].tolist())
    o.update()
    q = o.state()["queue"]
    assert sorted(q.tolist()) == sorted(set(range(1, 100)) - held)
