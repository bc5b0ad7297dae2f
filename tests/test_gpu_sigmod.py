"""The one-stage HotSketch (the artifact tree's sketch) on CUDA against its sequential CPU oracle, through the C ABI.

Identical (id, count) arrays go to both sides; per-lookup results (query, insert result) and the whole state
(slot ids, counts bit for bit, rows, the free-row FIFO in order, rows handed out, inserted mass) must be equal after
every call.  Counts are multiples of 1/256, so the inserted mass is exact in double whatever the order of addition."""
from pathlib import Path

import numpy as np
import pytest

from oracle.sigmod import OracleSigmod

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden" / "sigmod_stream.npz"


def same_state(a, b):
    bad = [k for k in ("val", "dic", "queue") if not np.array_equal(a[k], b[k])]
    if not np.array_equal(a["cnt"].view(np.uint32), b["cnt"].view(np.uint32)):
        bad.append("cnt")
    if a["num"] != b["num"] or a["tot"] != b["tot"]:
        bad.append(f"scalars {a['num']} {b['num']} {a['tot']} {b['tot']}")
    return bad


def test_golden_stream_from_the_reference():
    import cafe_b200
    g = np.load(GOLDEN)
    s = cafe_b200.SigmodSketch(int(g["lim"]), int(g["k"]), float(g["dr"]), max_lookups=g["ids"].shape[1])
    for c in range(g["ids"].shape[0]):
        assert np.array_equal(s.batch_query(g["ids"][c]), g["q0"][c]), f"call {c}: query before"
        m = s.batch_insert_val(g["ids"][c], g["v"][c]) if c % 3 else s.batch_insert(g["ids"][c])
        assert np.array_equal(m, g["mask"][c]), f"call {c}: insert result"
        assert np.array_equal(s.batch_query(g["ids"][c]), g["q1"][c]), f"call {c}: query after"
    want = dict(val=g["val"], cnt=g["cnt"], dic=g["dic"], queue=g["queue"], num=int(g["num"]), tot=float(g["tot"]))
    assert same_state(s.state(), want) == []


@pytest.mark.parametrize("lim,k,dr,calls,n,dom,zipf", [(50, 3, 0.8, 60, 200, 900, 1.3), (2000, 20, 0.99, 30, 4096, 100000, 1.1),
                                                       (128, 1, 0.5, 50, 333, 5000, 1.5), (40, 2, 0.9, 30, 3000, 60, 1.2),
                                                       (13505, 200, 0.99, 12, 65536, 10_000_000, 1.05)])
def test_random_streams_state_for_state(lim, k, dr, calls, n, dom, zipf):
    """Small sketches whose FIFO runs empty inside calls, decays at call boundaries, a 60-id domain (thousands of
    lookups per bucket and call), and a 65536-id call on a Kaggle-sized sketch."""
    import cafe_b200
    rng = np.random.default_rng(lim * 7 + k)
    o = OracleSigmod(lim, k, dr)
    s = cafe_b200.SigmodSketch(lim, k, dr, max_lookups=n)
    for c in range(calls):
        ids = np.minimum(rng.zipf(zipf, size=n), dom).astype(np.uint32)
        if c % 5 == 0:
            ids[::11] = 0
        v = (rng.integers(1, 2048, size=n) / 256.0).astype(np.float32)
        assert np.array_equal(s.batch_query(ids), o.batch_query(ids)), f"call {c}: query"
        if c % 4 == 3:
            assert np.array_equal(s.batch_insert(ids), o.batch_insert(ids)), f"call {c}: insert"
        else:
            assert np.array_equal(s.batch_insert_val(ids, v), o.batch_insert_val(ids, v)), f"call {c}: insert"
        assert same_state(s.state(), o.state()) == [], f"call {c}"
    assert s.state()["decays"] > 0 or lim >= 2000   # the small sketches pass their decay mass several times


def test_empty_call_and_checkpoint():
    import cafe_b200
    rng = np.random.default_rng(5)
    a = cafe_b200.SigmodSketch(200, 2, 0.9, max_lookups=512)
    o = OracleSigmod(200, 2, 0.9)
    for c in range(12):
        ids = np.minimum(rng.zipf(1.3, size=512), 3000).astype(np.uint32)
        a.batch_insert(ids); o.batch_insert(ids)
    assert a.batch_insert(np.zeros(0, np.uint32)).size == 0
    o.batch_insert(np.zeros(0, np.uint32))
    assert same_state(a.state(), o.state()) == []
    # a restored sketch rebuilds its free-row list the way update() does and continues identically
    b = cafe_b200.SigmodSketch(200, 2, 0.9, max_lookups=512)
    b.load_state(a.state())
    o.update()
    a.update()
    for c in range(6):
        ids = np.minimum(rng.zipf(1.3, size=512), 3000).astype(np.uint32)
        ma, mb, mo = a.batch_insert(ids), b.batch_insert(ids), o.batch_insert(ids)
        assert np.array_equal(ma, mo) and np.array_equal(mb, mo)
    assert same_state(b.state(), o.state()) == []


def test_module_steps_match_the_module_oracle():
    """SigmodSKEmbeddingBag for one field against the numpy module step over the one-stage sketch oracle: pooled rows
    exact at step 0 and within 1e-5 later, sketch state bit for bit (both sides get the kernel's importances), tables
    within 1e-5."""
    import torch
    import cafe_b200
    from oracle.module_oracle import ModuleOracle
    hotn, D, ncat, hash_size, B, off, lr = 300, 16, 5000, 40, 256, 7000, 0.1
    sk = cafe_b200.SigmodSketch(hotn, 3, 0.95, max_lookups=B)
    torch.manual_seed(0)
    wh = torch.nn.Parameter((torch.rand(hotn, D) * 2 - 1).cuda() * 0.05)
    m = cafe_b200.SigmodSKEmbeddingBag(0, hotn, sk, wh, "cuda", ncat, D, off, hash_size, False, max_batch=B)
    o = OracleSigmod(hotn, 3, 0.95)
    orc = ModuleOracle(o, wh.detach().cpu().numpy(), [m.weight_hash.detach().cpu().numpy()], [off], [hash_size])
    rng = np.random.default_rng(2)
    for step in range(25):
        ids = np.minimum(rng.zipf(1.2, size=B) - 1, ncat - 1).astype(np.int64)
        out = m(torch.from_numpy(ids), torch.arange(B))
        ref = orc.forward(ids[None, :])[:, 0]
        if step == 0:
            assert np.array_equal(out.detach().cpu().numpy(), ref)
        np.testing.assert_allclose(out.detach().cpu().numpy(), ref, rtol=1e-5, atol=1e-7)
        grad = (rng.standard_normal((B, D)) * 0.01).astype(np.float32)
        out.backward(torch.from_numpy(grad).cuda())
        mask = m.insert_grad(torch.from_numpy(ids), use_freq=(step % 5 == 4))
        imp = np.ones(B, np.float32) if step % 5 == 4 else ModuleOracle.importance(grad)
        if step % 5 != 4:
            # the sketch decides on the kernel's floats: feed the oracle the same ones
            g = torch.from_numpy(grad).cuda()
            k_imp = torch.empty(B, device="cuda")
            from cafe_b200 import _lib
            from cafe_b200.sketch import _stream
            _lib.check(sk.lib.cafe_grad_importance(m._ws.handle, g.data_ptr(), 0, D, 1, B, D, k_imp.data_ptr(), _stream()), "imp")
            np.testing.assert_allclose(k_imp.cpu().numpy(), imp, rtol=1e-5)
            imp = k_imp.cpu().numpy()
        masks, _ = orc.backward(ids[None, :], grad[:, None, :], lr, importance=imp[None, :])
        m.apply_update(lr)
        assert np.array_equal(mask.cpu().numpy(), masks[0]), f"step {step}: insert results"
        assert same_state(sk.state(), o.state()) == [], f"step {step}"
        np.testing.assert_allclose(wh.detach().cpu().numpy(), orc.wh, rtol=1e-5, atol=1e-7)
        np.testing.assert_allclose(m.weight_hash.detach().cpu().numpy(), orc.wc[0], rtol=1e-5, atol=1e-7)
