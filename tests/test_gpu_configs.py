"""Fused training steps at the shapes and batch sizes of the named configurations: Kaggle-shaped 26 fields / dim 16 /
batch 128, the Avazu-shaped large-hot-table regime (compress 0.1, hash-rate 0.7, 9 sketch fields, batch 4096) and
the Terabyte-shaped one (dim 128, batch 2048).  Bars as in tests/test_gpu_embed.py, with an absolute floor of 1e-6 on
table rows and pooled rows: at these batch sizes a hot id's row sums hundreds of gradient rows, in a different order
on the two sides, and elements whose sum nearly cancels cannot meet a purely relative bound."""
import numpy as np
import pytest

from oracle.hotsketch import OracleSketch, states_equal
from oracle.module_oracle import ModuleOracle

pytestmark = pytest.mark.gpu


def run_steps(cards, D, cr, hr, B, steps, s_zipf):
    import torch
    import cafe_b200
    from cafe_b200 import synthetic as S
    grp = cafe_b200.SKEmbeddingGroup(cards, D, cr, hr, 1, 1, 1.0000005, device="cuda", max_batch=B, lr=0.1, seed=2)
    sk = OracleSketch(grp.hotn, 1, 1, 1.0000005)
    orc = ModuleOracle(sk, grp.weight_high.detach().cpu().numpy(), [w.detach().cpu().numpy() for w in grp.weight_hash],
                       grp.f_offsets, grp.hash_sizes)
    F = len(cards)
    for s in range(steps):
        ids = S.batch_ids(cards, B, s_zipf, 7, s)
        out = grp(torch.from_numpy(ids))
        ref = orc.forward(ids)
        np.testing.assert_allclose(out.detach().cpu().numpy(), ref, rtol=1e-5, atol=1e-6)
        grad = S.gradients(B, F, D, 7, s)
        g = torch.from_numpy(grad).cuda()
        imp = grp._fields.importance(g, D, F * D, B).view(F, B).cpu().numpy()
        out.backward(g)
        orc.backward(ids, grad, grp.lr, importance=imp)
        assert states_equal(sk.state(), grp.sketch.state()) == [], f"step {s}"
        np.testing.assert_allclose(grp.weight_high.detach().cpu().numpy(), orc.wh, rtol=1e-5, atol=1e-6)
    for f in range(F):
        np.testing.assert_allclose(grp.weight_hash[f].detach().cpu().numpy(), orc.wc[f], rtol=1e-5, atol=1e-6)
    return grp.sketch.stats()


def test_kaggle_shape_26_fields_dim16_batch128():
    from cafe_b200 import sizing, synthetic as S
    assert sizing.hot_rows(sum(S.KAGGLE_CARDS), 0.001, 0.3, 16) == 13505
    st = run_steps(S.KAGGLE_CARDS, 16, 0.001, 0.3, 128, 40, 1.1)
    assert st["resets"] > 0 and st["seq_fallbacks"] == 0


def test_avazu_shape_large_hot_table_regime():
    from cafe_b200 import sizing, synthetic as S
    cards = [n for n in S.AVAZU_CARDS if sizing.is_sketch_field(n, 0.1)]
    assert len(cards) == 9
    run_steps(cards, 16, 0.1, 0.7, 4096, 8, 1.0)


def test_terabyte_shape_dim128():
    from cafe_b200 import synthetic as S
    run_steps(S.TERABYTE_CARDS, 128, 0.001, 0.3, 2048, 8, 1.1)
