"""The peer-memory exchange entry points on ONE GPU: two ranks are emulated one after the other with
buffers that all live on this device, so the address arithmetic of cafe_shard_scatter_ids,
cafe_embed_forward_sharded, cafe_shard_pull_importance and cafe_embed_backward_imp is compared with
the unsharded entry points (no kernel waits for another, so nothing can hang)."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _ptrs(tensors, offs=None, size=4):
    offs = offs or [0] * len(tensors)
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() + o * size for t, o in zip(tensors, offs)])


def test_emulated_two_rank_exchange_matches_unsharded_calls():
    import torch
    import cafe_b200
    from cafe_b200 import _lib, sizing
    from cafe_b200.sharded import FieldShardPlan
    from cafe_b200.sketch import _stream
    lib = cafe_b200.load_library()
    G, D, Bl = 2, 16, 96
    cards = [5000, 120000, 37, 800000, 2500]
    F = len(cards)
    offs = sizing.field_offsets(cards)
    plans = [FieldShardPlan(F, G, r) for r in range(G)]
    rng = np.random.default_rng(0)
    ids_local = [torch.from_numpy(np.stack([rng.integers(0, n, Bl) for n in cards]).astype(np.int64)).cuda() for _ in range(G)]

    # --- ids: every rank stores its slice into the owners' buffers
    fmax = max(plans[0].counts)
    owner_ids = [torch.full((fmax * G * Bl,), -1, dtype=torch.int64, device="cuda") for _ in range(G)]
    for r in range(G):
        assert lib.cafe_shard_scatter_ids(ids_local[r].data_ptr(), F, Bl, G, r, _ptrs(owner_ids, size=8), _stream()) == 0
    for g in range(G):
        own = owner_ids[g][:plans[g].counts[g] * G * Bl].view(plans[g].counts[g], G * Bl)
        for j, f in enumerate(plans[g].local_fields):
            for r in range(G):
                assert torch.equal(own[j, r * Bl:(r + 1) * Bl], ids_local[r][f])

    # --- forward: owners store pooled rows straight into the consumers' blocked buffers
    groups, outs = [], []
    pooled = [torch.zeros(Bl * F * D, device="cuda") for _ in range(G)]
    block_off = [Bl * D * sum(plans[0].counts[:r]) for r in range(G)]
    saved = []
    for g in range(G):
        mine = plans[g].local_fields
        grp = cafe_b200.SKEmbeddingGroup([cards[f] for f in mine], D, 0.01, 0.3, 1, 1, 1.0000005, device="cuda",
                                         max_batch=G * Bl, lr=0.1, f_offsets=[offs[f] for f in mine], seed=3 + g)
        groups.append(grp)
        Fg = len(mine)
        own = owner_ids[g][:Fg * G * Bl]
        f = grp._fields
        wp, hp = f.ptrs()
        gid = torch.empty(Fg * G * Bl, dtype=torch.int32, device="cuda")
        row = torch.empty_like(gid)
        rc = lib.cafe_embed_forward_sharded(grp.sketch.handle, own.data_ptr(), 1, Fg, G * Bl, f.f_offset, f.hash_size, wp, hp,
                                            f.hotn, D, _ptrs(pooled, [block_off[g]] * G), G, Bl, D, Fg * D, gid.data_ptr(),
                                            row.data_ptr(), _stream())
        assert rc == 0
        ref = torch.empty(G * Bl, Fg, D, device="cuda")
        gid2, row2 = f.forward(own, ref, D, Fg * D)
        assert torch.equal(gid, gid2) and torch.equal(row, row2)
        outs.append(ref)
        saved.append((own, gid, row))
    for r in range(G):
        blocks = plans[r].blocks(pooled[r], Bl, D)
        for g in range(G):
            assert torch.equal(blocks[g], outs[g][r * Bl:(r + 1) * Bl])

    # --- backward: owners pull gradient rows from the consumers' buffers and get the importance
    gradc = [torch.randn(Bl * F * D, device="cuda") * 0.01 for _ in range(G)]
    # (the same exchange driven by the consumers: every rank stores its rows into the owners' buffers)
    owner_grad = [torch.zeros(G * Bl * fmax * D, device="cuda") for _ in range(G)]
    for r in range(G):
        assert lib.cafe_shard_push_grads(gradc[r].data_ptr(), F, Bl, D, G, r, _ptrs(owner_grad), _stream()) == 0
    for g in range(G):
        Fg = groups[g].num_fields
        want = torch.cat([plans[r].blocks(gradc[r], Bl, D)[g] for r in range(G)], dim=0)
        assert torch.equal(owner_grad[g][:G * Bl * Fg * D].view(G * Bl, Fg, D), want)
    for g in range(G):
        grp = groups[g]
        Fg = grp.num_fields
        local = torch.zeros(G * Bl * Fg * D, device="cuda")
        imp = torch.zeros(G * Bl * Fg, device="cuda")
        rc = lib.cafe_shard_pull_importance(grp.sketch.handle, _ptrs(gradc, [block_off[g]] * G), G, Bl, Fg, D, D, Fg * D,
                                            local.data_ptr(), imp.data_ptr(), _stream())
        assert rc == 0
        want = torch.cat([plans[r].blocks(gradc[r], Bl, D)[g] for r in range(G)], dim=0)   # [G*Bl, Fg, D]
        assert torch.equal(local.view(G * Bl, Fg, D), want)
        imp_ref = grp._fields.importance(want.contiguous(), D, Fg * D, G * Bl)
        np.testing.assert_allclose(imp.cpu().numpy(), imp_ref.cpu().numpy(), rtol=1e-6)
        # the update through the two-call form equals the one-call backward on a twin group
        twin = cafe_b200.SKEmbeddingGroup([cards[f] for f in plans[g].local_fields], D, 0.01, 0.3, 1, 1, 1.0000005,
                                          device="cuda", max_batch=G * Bl, lr=0.1,
                                          f_offsets=[offs[f] for f in plans[g].local_fields], seed=3 + g)
        own, gid, row = saved[g]
        f = grp._fields
        wp, hp = f.ptrs()
        rc = lib.cafe_embed_backward_imp(grp.sketch.handle, local.data_ptr(), D, Fg * D, imp.data_ptr(), own.data_ptr(), 1,
                                         gid.data_ptr(), row.data_ptr(), Fg, G * Bl, f.f_offset, f.hash_size, wp, hp, f.hotn, D,
                                         0.1, 0, None, _stream())
        assert rc in (0, 4, 5)
        ref = torch.empty(G * Bl, Fg, D, device="cuda")
        g2, r2 = twin._fields.forward(own, ref, D, Fg * D)
        twin._fields.backward(want.contiguous(), D, Fg * D, own, g2, r2, G * Bl, 0.1, 0)
        from oracle.hotsketch import states_equal
        assert states_equal(grp.sketch.state(), twin.sketch.state()) == []
        assert torch.equal(grp.weight_high, twin.weight_high)
        for a, b in zip(grp.weight_hash, twin.weight_hash):
            assert torch.equal(a, b)
