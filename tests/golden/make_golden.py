"""Generates the golden fixtures of this folder from the reference itself.

Run in a container that has the reference checkout (it compiles tricks/sketch.cpp through
oracle/build_ref.sh):   python tests/golden/make_golden.py

Outputs
  kat_hashes.json      -- FNV-1a-64 of all query/insert/query results of three seeded streams, the
                          number of newly-hot results, the number of hot query results and a SHA-256
                          of the final sketch state, all produced by the compiled reference.
  small_stream.npz     -- a small seeded stream (ids, importances) with the reference's per-call
                          outputs and its final state arrays, for tests that run where the reference
                          checkout is absent.
"""
import hashlib
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))

from kat_stream import KATS, SplitMix64, kat_call, run_kat  # noqa: E402
from oracle.hotsketch import ReferenceSketch  # noqa: E402

STATE_KEYS = ["main_val", "main_cnt", "main_dic", "main_flip", "lru_val", "lru_cnt", "lru_dic", "lru_t",
              "lru_flip", "queue"]


def state_digest(st: dict) -> str:
    h = hashlib.sha256()
    for k in STATE_KEYS:
        h.update(np.ascontiguousarray(st[k]).tobytes())
    h.update(json.dumps([st["thr_bits"], st["real_n"], st["num"], st["t"], st["gflip"]]).encode())
    return h.hexdigest()


def main():
    out = []
    for k in KATS:
        s = ReferenceSketch(k["lim"], k["thr"], 1, k["alpha"])
        fnv, newhot, hotq = run_kat(s, k["calls"], k["n"], k["dom"])
        st = s.state()
        out.append(dict(k, fnv1a64=fnv, newhot=newhot, hotq=hotq, state_sha256=state_digest(st),
                        thr_bits=st["thr_bits"], real_n=st["real_n"], num=st["num"], t=st["t"],
                        queue_len=int(st["queue"].size)))
        print(out[-1])
    (HERE / "kat_hashes.json").write_text(json.dumps(out, indent=1) + "\n")

    # small stream with full outputs: lim 200, threshold 1, 40 calls of 96 ids, alpha large enough
    # to flip once, domain small enough to force promotions, evictions and resets
    lim, thr, alpha, calls, n, dom = 200, 1, 1.3, 40, 96, 3000
    s = ReferenceSketch(lim, thr, 1, alpha)
    rng = SplitMix64(7)
    ids_all, v_all, q0_all, m_all, q1_all = [], [], [], [], []
    for _ in range(calls):
        ids, v = kat_call(rng, n, dom)
        ids_all.append(ids)
        v_all.append(v)
        q0_all.append(s.batch_query(ids))
        m_all.append(s.batch_insert_val(ids, v))
        q1_all.append(s.batch_query(ids))
    st = s.state()
    np.savez_compressed(
        HERE / "small_stream.npz", lim=lim, thr=thr, alpha=alpha, ids=np.stack(ids_all), v=np.stack(v_all),
        q0=np.stack(q0_all), mask=np.stack(m_all), q1=np.stack(q1_all),
        scalars=np.array([st["thr_bits"], st["real_n"], st["num"], st["t"], st["gflip"]], np.int64),
        **{k: st[k] for k in STATE_KEYS})
    print("small_stream: newhot", int(np.stack(m_all).sum()), "thr_bits", st["thr_bits"], "real_n", st["real_n"])


if __name__ == "__main__":
    main()
