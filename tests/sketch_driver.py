"""Shared driver: feeds seeded streams to the sequential oracle and to an implementation under test
(CPU emulation of the device engine, or the CUDA library) and compares outputs and full state."""
import numpy as np

from kat_stream import SplitMix64, kat_call
from oracle.hotsketch import OracleSketch, states_equal


def drive(factory, lim, thr, alpha, calls, n, dom, fuse, parallel=True, seed=7, unit=False, zero_ids=False, window=None,
          round_cap=None, ragged=False, size_jobs_by_rate=True):
    o = OracleSketch(lim, thr, 1, alpha)
    e = factory(lim, thr, 1, alpha, max(1, n * fuse), parallel)
    if window:
        e.set_window(window)
    if round_cap:
        e.set_round_cap(round_cap)
    if not size_jobs_by_rate:
        e.set_job_sizing(False)   # (host emulation only) every job takes all its segments: re-fits cut most of them short
    rng = SplitMix64(seed)
    for c in range(0, calls, fuse):
        idl, vl, ml, pl, off = [], [], [], [], [0]
        for f in range(fuse):
            m = n if not ragged else (0 if (c + f) % 5 == 2 else 1 + (c * 7 + f * 13) % n)
            ids, v = kat_call(rng, n, dom)
            ids, v = ids[:m], v[:m]
            if zero_ids and m:
                ids[::7] = 0
            idl.append(ids)
            vl.append(v)
            q0 = o.batch_query(ids)
            assert np.array_equal(e.batch_query(ids), q0) or f > 0  # state before the fused job only
            ml.append(o.batch_insert_val(ids, None if unit else v))
            q = o.batch_query(ids)
            pl.append(np.where((ml[-1] == 1) & (q < 0), -q, 0))
            off.append(off[-1] + m)
        ids, v = np.concatenate(idl), np.concatenate(vl)
        m = e.insert_segments(ids, None if unit else v, off)
        assert e.last_rc in (0, 4), e.last_rc
        assert np.array_equal(m, np.concatenate(ml)), f"mask differs in job at call {c}"
        assert np.array_equal(np.where(m == 1, e.last_post_row, 0), np.concatenate(pl)), f"post rows differ at call {c}"
        assert states_equal(o.state(), e.state()) == [], f"state differs after job at call {c}"
        assert np.array_equal(e.batch_query(ids), o.batch_query(ids))
    return e.stats()


