"""Generates sigmod_stream.npz from the reference's one-stage sketch (ArtifactEvaluation/embeddings/sketch.cpp,
compiled by oracle/build_ref.sh): a seeded stream of calls with the reference's per-call outputs and final state.

    python tests/golden/make_golden_sigmod.py

The stream reaches every path: hits with and without a free row left, the sorted-slot bubbling, empty-slot fills,
replacement of the last slot, and several decays (small threshold, decay rate 0.9)."""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
from oracle.sigmod import ReferenceSigmod  # noqa: E402


def stream(calls=120, n=512, dom=6000, seed=11):
    rng = np.random.default_rng(seed)
    ids = np.minimum(rng.zipf(1.25, size=(calls, n)), dom).astype(np.uint32)
    ids[::9, ::5] = 0                                     # id 0 is an ordinary id here
    v = (rng.integers(1, 1024, size=(calls, n)) / 256.0).astype(np.float32)   # sums stay exact in double
    return ids, v


def main():
    lim, k, dr = 300, 6, 0.9
    ids, v = stream()
    r = ReferenceSigmod(lim, k, dr)
    q0, m, q1 = [], [], []
    for c in range(ids.shape[0]):
        q0.append(r.batch_query(ids[c]))
        m.append(r.batch_insert_val(ids[c], v[c]) if c % 3 else r.batch_insert(ids[c]))
        q1.append(r.batch_query(ids[c]))
    st = r.state()
    np.savez_compressed(HERE / "sigmod_stream.npz", lim=lim, k=k, dr=dr, ids=ids, v=v, q0=np.stack(q0), mask=np.stack(m),
                        q1=np.stack(q1), val=st["val"], cnt=st["cnt"], dic=st["dic"], queue=st["queue"], num=st["num"], tot=st["tot"])
    print("written", HERE / "sigmod_stream.npz", "num", st["num"], "queue", len(st["queue"]), "tot", st["tot"])


if __name__ == "__main__":
    main()
