"""The numpy restatement of the module step against the fixture recorded from the reference's own
SKEmbeddingBag class (tests/golden/make_module_golden.py), on CPU and -- marked gpu -- the CUDA path
against the same fixture."""
from pathlib import Path

import numpy as np
import pytest

from oracle.hotsketch import OracleSketch
from oracle.module_oracle import ModuleOracle

G = np.load(Path(__file__).resolve().parent / "golden" / "module_step.npz")
STATE_KEYS = ["main_val", "main_cnt", "main_dic", "main_flip", "lru_val", "lru_cnt", "lru_dic", "lru_t", "lru_flip",
              "queue"]


def _state_matches(st):
    for k in STATE_KEYS:
        a, b = st[k], G[k]
        if a.dtype == np.float32:
            a, b = a.view(np.uint32), b.view(np.uint32)
        assert np.array_equal(a, b), k
    assert [st["thr_bits"], st["real_n"], st["num"], st["t"], st["gflip"]] == list(G["scalars"])


def test_numpy_restatement_reproduces_reference_module():
    sk = OracleSketch(int(G["hotn"]), float(G["thr"]), 0, 1.0000005)
    orc = ModuleOracle(sk, G["wh0"], [G["wc0"]], [0], [int(G["hash_size"])])
    for s in range(G["ids"].shape[0]):
        ids = G["ids"][s][None]
        out = orc.forward(ids)
        np.testing.assert_allclose(out[:, 0], G["out"][s], rtol=1e-5, atol=1e-7)
        imp = ModuleOracle.importance(G["grad"][s])
        np.testing.assert_allclose(imp, G["imp"][s], rtol=1e-6)
        masks, _ = orc.backward(ids, G["grad"][s][:, None], float(G["lr"]), importance=G["imp"][s][None])
        assert int(masks.sum()) == int(G["newhot"][s])
    np.testing.assert_allclose(orc.wh, G["wh"], rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(orc.wc[0], G["wc"], rtol=1e-5, atol=1e-7)
    _state_matches(sk.state())


@pytest.mark.gpu
def test_cuda_module_reproduces_reference_module():
    import torch
    import cafe_b200
    hotn, D, hs, lr = int(G["hotn"]), int(G["D"]), int(G["hash_size"]), float(G["lr"])
    B = G["ids"].shape[1]
    sk = cafe_b200.HotSketch(hotn, float(G["thr"]), 0, 1.0000005, max_lookups=B)
    wh = torch.nn.Parameter(torch.from_numpy(G["wh0"]).cuda())
    m = cafe_b200.SKEmbeddingBag(0, hotn, sk, wh, "cuda", int(G["ncat"]), D, 0, hs)
    with torch.no_grad():
        m.weight_hash.copy_(torch.from_numpy(G["wc0"]))
    for s in range(G["ids"].shape[0]):
        ids = torch.from_numpy(G["ids"][s])
        out = m(ids, torch.arange(B))
        np.testing.assert_allclose(out.detach().cpu().numpy(), G["out"][s], rtol=1e-5, atol=1e-7)
        out.backward(torch.from_numpy(G["grad"][s]).cuda())
        imp = m._fields.importance(m._saved["grad"], 0, D, B)
        np.testing.assert_allclose(imp.cpu().numpy(), G["imp"][s], rtol=1e-5)
        # same floats into the sketch as the reference used, so that its state can be compared exactly
        mask, post = sk.insert(m._saved["gid"], torch.from_numpy(G["imp"][s]).cuda(), [0, B])
        assert int(mask.sum()) == int(G["newhot"][s])
        m._fields.migrate(m._saved["ids"], mask, post, B)
        m.apply_update(lr)
    np.testing.assert_allclose(wh.detach().cpu().numpy(), G["wh"], rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(m.weight_hash.detach().cpu().numpy(), G["wc"], rtol=1e-5, atol=1e-7)
    _state_matches(sk.state())
