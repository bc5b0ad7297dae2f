"""Parity at the sizes that are benchmarked: the fused step of the microbenchmark configuration (26 fields x 65536
ids, dim 128, 665 600 hot rows) and the Terabyte-shaped sharding configuration's sketch regime (13 733 hot rows fed
65536-id calls: about five lookups per sketch slot per call, the regime with the most rounds per job).

Bars: sketch state, insert masks and row choices bit for bit (both sides get the kernel's importance floats); pooled
rows are copies and must match to 1e-5 relative; updated table rows to 1e-5 relative with an absolute floor of 1e-6
(fp32 sums of up to several thousand gradient rows per hot id, added in a different order on the two sides)."""
import numpy as np
import pytest

from oracle.hotsketch import OracleSketch, states_equal
from oracle.module_oracle import ModuleOracle

pytestmark = pytest.mark.gpu


def fused_steps(cards, D, cr, hr, B, steps, ids_of_step, seed=11, atol=1e-6):
    import torch
    import cafe_b200
    grp = cafe_b200.SKEmbeddingGroup(cards, D, cr, hr, 1, 1, 1.0000005, device="cuda", max_batch=B, lr=0.1, seed=seed)
    sk = OracleSketch(grp.hotn, 1, 1, 1.0000005)
    orc = ModuleOracle(sk, grp.weight_high.detach().cpu().numpy(), [w.detach().cpu().numpy() for w in grp.weight_hash],
                       grp.f_offsets, grp.hash_sizes)
    F = len(cards)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    for s in range(steps):
        ids = ids_of_step(s)
        out = grp(torch.from_numpy(ids))
        ref = orc.forward(ids)
        np.testing.assert_allclose(out.detach().cpu().numpy(), ref, rtol=1e-5, atol=atol, err_msg=f"step {s}: pooled rows")
        rows = grp.last_rows.cpu().numpy()
        for f in range(F):
            hot, rh, rc = orc.rows[f]
            assert np.array_equal(rows[f] < 0, hot), f"step {s} field {f}: hot flags"
            assert np.array_equal(np.where(hot, -rows[f], rows[f]), np.where(hot, rh, rc)), f"step {s} field {f}: rows"
        g = torch.randn(B, F, D, device="cuda", generator=gen) * 0.01   # drawn on the device, copied to the oracle
        grad = g.cpu().numpy()
        imp = grp._fields.importance(g, D, F * D, B).view(F, B).cpu().numpy()
        out.backward(g)
        del out, g
        orc.backward(ids, grad, grp.lr, importance=imp)
        assert states_equal(sk.state(), grp.sketch.state()) == [], f"step {s}: sketch state"
        np.testing.assert_allclose(grp.weight_high.detach().cpu().numpy(), orc.wh, rtol=1e-5, atol=atol, err_msg=f"step {s}: hot table")
    for f in range(F):
        np.testing.assert_allclose(grp.weight_hash[f].detach().cpu().numpy(), orc.wc[f], rtol=1e-5, atol=atol,
                                   err_msg=f"hash table {f}")
    return grp.sketch.stats()


def test_microbenchmark_configuration_fused_steps():
    """configs[1] at full size: four fused steps from the cold start (which includes its threshold re-fits)."""
    from cafe_b200 import sizing, synthetic as S
    cards = S.MICRO_CARDS
    assert sizing.hot_rows(sum(cards), 0.001, 0.3, 128) == 665600
    st = fused_steps(cards, 128, 0.001, 0.3, 65536, 4, lambda s: S.batch_ids(cards, 65536, 1.05, 2024, s))
    assert st["seq_fallbacks"] == 0 and st["resets"] > 0
    assert st["lookups"] == 4 * 26 * 65536
    print("microbenchmark shape:", st)


def test_sharding_configuration_sketch_regime():
    """configs[3]'s sketch: Terabyte cardinalities at compress 1e-4 / hash-rate 0.2 give 13 733 hot rows; 52 calls of
    65536 ids each (two steps of 26 fields), the drifting id stream across a re-permutation, sketch only."""
    import torch
    import cafe_b200
    from cafe_b200 import sizing, synthetic as S
    cards = S.TERABYTE_CARDS
    lim = sizing.hot_rows(sum(cards), 0.0001, 0.2, 128)
    assert lim == 13733
    B, F = 65536, len(cards)
    off = sizing.field_offsets(cards)
    sk = cafe_b200.HotSketch(lim, 1, 1, 1.0000005, max_lookups=F * B)
    o = OracleSketch(lim, 1, 1, 1.0000005)
    rng = np.random.default_rng(3)
    for step, wstep in enumerate((900, 1000)):       # the second one lies behind the first re-permutation
        ids = S.drift_batch_ids(cards, B, 2024, wstep)
        gid = np.stack([(ids[f] + off[f]).astype(np.uint32) for f in range(F)])
        imp = rng.random((F, B)).astype(np.float32) * 2
        imp *= (B / imp.sum(axis=1, keepdims=True)).astype(np.float32)    # mean 1 per field, like the importance
        want_m, want_row = [], []
        for f in range(F):
            m = o.batch_insert_val(gid[f], imp[f])
            q = o.batch_query(gid[f])
            want_m.append(m)
            want_row.append(np.where((m == 1) & (q < 0), -q, 0))
        t = torch.from_numpy(gid.reshape(-1).view(np.int32)).cuda()
        mask, post = sk.insert(t, torch.from_numpy(imp.reshape(-1)).cuda(), [f * B for f in range(F + 1)])
        mask, post = mask.cpu().numpy(), post.cpu().numpy()
        assert np.array_equal(mask, np.concatenate(want_m)), f"step {step}: insert results"
        assert np.array_equal(np.where(mask == 1, post, 0), np.concatenate(want_row)), f"step {step}: post-insert rows"
        assert states_equal(o.state(), sk.state()) == [], f"step {step}: sketch state"
    st = sk.stats()
    assert st["seq_fallbacks"] == 0, st
    assert st["calls"] == 52
    print("sharding configuration sketch regime: max rounds per job", st["max_rounds"], st)


def test_sharding_configuration_fused_steps():
    """configs[3] un-sharded (all 26 Terabyte fields on one GPU), global batch 65536, dim 128: two fused steps.

    The tables are tiny here (at most 800 hash rows per field, 13 733 hot rows), so one row sums the gradient rows
    of up to several thousand lookups of a 65536-id call.  Each side adds them in fp32 in its own order; with partial
    sums near 1 and K of a few thousand, sqrt(K) * 2^-24 * |partial sum| per side is several 1e-6, hence the absolute
    floor of 2e-5 beside the 1e-5 relative bound."""
    from cafe_b200 import synthetic as S
    cards = S.TERABYTE_CARDS
    st = fused_steps(cards, 128, 0.0001, 0.2, 65536, 2, lambda s: S.drift_batch_ids(cards, 65536, 2024, 1000 * s), atol=2e-5)
    assert st["seq_fallbacks"] == 0
