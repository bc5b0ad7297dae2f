"""Parity of the CUDA SKEmbeddingBag path with the CPU restatement of the reference's module step.

Tolerances: row choices, insert masks and the sketch state are compared bit for bit (both sides get
the same importance floats); pooled embeddings are copies and compared exactly; updated rows and
importances are compared at 1e-5 relative (fp32, different summation order)."""
import numpy as np
import pytest

from oracle.hotsketch import OracleSketch, states_equal
from oracle.module_oracle import ModuleOracle

pytestmark = pytest.mark.gpu
RTOL = 1e-5


def zipf_ids(rng, n, size, s=1.05):
    r = np.minimum(rng.zipf(s + 0.25, size=size) - 1, n - 1)   # heavy head, many duplicates
    perm_mul = 2654435761 % n or 1
    return ((r.astype(np.int64) * perm_mul + 12345) % n).astype(np.int64)


def make_pair(cards, D, cr, hr, thr=1, alpha=1.0000005, B=256, seed=0, lr=0.1, mode=None):
    import torch
    import cafe_b200
    grp = cafe_b200.SKEmbeddingGroup(cards, D, cr, hr, thr, 1, alpha, device="cuda", max_batch=B, lr=lr, seed=seed,
                                     insert_mode=cafe_b200.INSERT_PARALLEL if mode is None else mode)
    sk = OracleSketch(grp.hotn, thr, 1, alpha)
    orc = ModuleOracle(sk, grp.weight_high.detach().cpu().numpy(), [w.detach().cpu().numpy() for w in grp.weight_hash],
                       grp.f_offsets, grp.hash_sizes)
    return grp, orc, sk


def close(a, b, what):
    np.testing.assert_allclose(a, b, rtol=RTOL, atol=1e-7, err_msg=what)


@pytest.mark.parametrize("D,B", [(16, 128), (128, 256), (64, 96), (32, 33)])
def test_training_steps_match_oracle(D, B):
    import torch
    cards = [5000, 120000, 37, 800000, 2500]
    grp, orc, sk = make_pair(cards, D, 0.01, 0.3, B=B)
    rng = np.random.default_rng(D + B)
    F = len(cards)
    for step in range(12):
        ids = np.stack([zipf_ids(rng, n, B) for n in cards])
        t_ids = torch.from_numpy(ids)                      # CPU int64, as the reference's loaders give
        out = grp(t_ids)
        ref = orc.forward(ids)
        # gathered rows are copies: exact while the tables are (step 0), within the update tolerance later
        if step == 0:
            assert np.array_equal(out.detach().cpu().numpy(), ref), "step 0: pooled embeddings"
        close(out.detach().cpu().numpy(), ref, f"step {step}: pooled embeddings")
        rows = grp.last_rows.cpu().numpy()
        for f in range(F):
            hot, rh, rc = orc.rows[f]
            assert np.array_equal(rows[f] < 0, hot) and np.array_equal(np.where(hot, -rows[f], rows[f]), np.where(hot, rh, rc))
        grad = (rng.standard_normal((B, F, D)) * 0.01).astype(np.float32)
        g = torch.from_numpy(grad).cuda()
        imp = grp._fields.importance(g, D, F * D, B).view(F, B).cpu().numpy()
        for f in range(F):
            close(imp[f], ModuleOracle.importance(grad[:, f]), f"step {step}: importance of field {f}")
        out.backward(g)
        masks, _ = orc.backward(ids, grad, grp.lr, importance=imp)
        assert states_equal(sk.state(), grp.sketch.state()) == [], f"step {step}: sketch state"
        close(grp.weight_high.detach().cpu().numpy(), orc.wh, f"step {step}: hot table")
        for f in range(F):
            close(grp.weight_hash[f].detach().cpu().numpy(), orc.wc[f], f"step {step}: hash table {f}")
    st = grp.sketch.stats()
    assert st["lookups"] == 12 * F * B and st["seq_fallbacks"] == 0


def test_sequential_insert_mode_gives_same_step():
    import torch
    import cafe_b200
    cards = [3000, 90000, 40000]
    a, orc, sk = make_pair(cards, 16, 0.01, 0.3, B=200, mode=cafe_b200.INSERT_SEQUENTIAL)
    rng = np.random.default_rng(5)
    for step in range(6):
        ids = np.stack([zipf_ids(rng, n, 200) for n in cards])
        out = a(torch.from_numpy(ids))
        orc.forward(ids)
        grad = (rng.standard_normal((200, 3, 16)) * 0.01).astype(np.float32)
        g = torch.from_numpy(grad).cuda()
        imp = a._fields.importance(g, 16, 48, 200).view(3, 200).cpu().numpy()
        out.backward(g)
        orc.backward(ids, grad, a.lr, importance=imp)
        assert states_equal(sk.state(), a.sketch.state()) == []
        close(a.weight_high.detach().cpu().numpy(), orc.wh, "hot table")


def test_scatter_long_duplicate_runs():
    """One id repeated thousands of times: its row's gradient spans many 32-lookup chunks."""
    import torch
    grp, orc, sk = make_pair([50, 1000], 128, 0.5, 0.5, thr=500, B=4096, lr=0.5)
    rng = np.random.default_rng(9)
    ids = np.stack([np.where(rng.random(4096) < 0.8, 7, rng.integers(0, 50, 4096)),
                    np.where(rng.random(4096) < 0.5, 3, rng.integers(0, 1000, 4096))]).astype(np.int64)
    out = grp(torch.from_numpy(ids).cuda())
    orc.forward(ids)
    grad = rng.standard_normal((4096, 2, 128)).astype(np.float32)
    out.backward(torch.from_numpy(grad).cuda())
    # float64 reference of the summed update, compared at fp32 accumulation tolerance
    for f in range(2):
        hot, rh, rc = orc.rows[f]
        assert not hot.any()
        acc = np.zeros(orc.wc[f].shape, np.float64)
        np.add.at(acc, rc, grad[:, f].astype(np.float64))
        want = orc.wc[f].astype(np.float64) - 0.5 * acc
        np.testing.assert_allclose(grp.weight_hash[f].detach().cpu().numpy(), want, rtol=1e-4, atol=2e-3)


def test_empty_batch_and_bad_arguments():
    import torch
    import cafe_b200
    grp, _, _ = make_pair([3000, 5000], 16, 0.01, 0.3, B=64)
    out = grp(torch.zeros(2, 0, dtype=torch.int64))
    assert out.shape == (0, 2, 16)
    with pytest.raises(ValueError):
        grp(torch.zeros(3, 4, dtype=torch.int64))
    with pytest.raises(ValueError):
        grp(torch.zeros(2, 65, dtype=torch.int64))      # beyond max_batch
    with pytest.raises(TypeError):
        grp(torch.zeros(2, 4, dtype=torch.float32))
    with pytest.raises(ValueError):
        cafe_b200.SKEmbeddingGroup([100], 16, 0.5, 0.3, device="cpu")


def test_dropin_module_matches_group_and_reference_call_pattern():
    """SKEmbeddingBag built and driven the way DLRM_Net does it (dlrm_s_pytorch.py:309-322, 438-449,
    653-659, 734-738, 1653-1658), with ids on the CPU and offsets = arange(B)."""
    import torch
    import cafe_b200
    from cafe_b200 import sizing
    cards, D, cr, hr, B, lr = [4000, 70000, 900], 16, 0.01, 0.3, 128, 0.1
    hotn = sizing.hot_rows(sum(cards), cr, hr, D)
    lib = cafe_b200.load_library()
    lib.init(hotn, 1, 1, 1.0000005)
    torch.manual_seed(0)
    weight_high = torch.nn.Parameter((torch.rand(hotn, D) * 0.02 - 0.01).cuda())
    offs = sizing.field_offsets(cards)
    mods = [cafe_b200.SKEmbeddingBag(k, hotn, lib, weight_high, "cuda", n, D, offs[k], sizing.hash_rows(n, cr, hr))
            for k, n in enumerate(cards)]
    dense = torch.nn.Linear(D * len(cards), 1).cuda()
    opt = torch.optim.SGD([weight_high] + [m.weight_hash for m in mods] + list(dense.parameters()), lr=lr)
    cafe_b200.attach_optimizer(opt, mods)
    sk = OracleSketch(hotn, 1, 1, 1.0000005)
    orc = ModuleOracle(sk, weight_high.detach().cpu().numpy(), [m.weight_hash.detach().cpu().numpy() for m in mods],
                       offs, [m.hash_size for m in mods])
    rng = np.random.default_rng(2)
    off_t = torch.arange(B)
    for step in range(8):
        ids = np.stack([zipf_ids(rng, n, B) for n in cards])
        outs = [m(torch.from_numpy(ids[k]), off_t) for k, m in enumerate(mods)]
        ref = orc.forward(ids)
        for k in range(3):
            close(outs[k].detach().cpu().numpy(), ref[:, k], f"step {step}: pooled embeddings of field {k}")
        for o in outs:
            o.retain_grad()
        loss = dense(torch.cat(outs, dim=1)).sigmoid().mean()
        opt.zero_grad()
        loss.backward()
        grad = np.stack([o.grad.cpu().numpy() for o in outs], axis=1)
        imps = []
        for k, m in enumerate(mods):
            imps.append(m._fields.importance(m._saved["grad"], 0, D, B).cpu().numpy())
            m.insert_grad(torch.from_numpy(ids[k]))
        opt.step()
        orc.backward(ids, grad, lr, importance=np.stack(imps))
        assert states_equal(sk.state(), mods[0].sketch.state()) == [], f"step {step}"
        close(weight_high.detach().cpu().numpy(), orc.wh, f"step {step}: hot table")
        for k, m in enumerate(mods):
            close(m.weight_hash.detach().cpu().numpy(), orc.wc[k], f"step {step}: hash table {k}")
        assert weight_high.grad is None and all(m.weight_hash.grad is None for m in mods)


def test_reference_compatible_sparse_gradients():
    """fused_update=False: the module returns the sparse gradients torch.optim.SGD expects."""
    import torch
    import cafe_b200
    torch.manual_seed(11)
    hotn, D, B = 200, 16, 64
    sk = cafe_b200.HotSketch(hotn, 1, 1, 1.0000005, max_lookups=B)
    wh = torch.nn.Parameter(torch.randn(hotn, D).cuda() * 0.01)
    m = cafe_b200.SKEmbeddingBag(0, hotn, sk, wh, "cuda", 5000, D, 0, 30, fused_update=False)
    opt = torch.optim.SGD([wh, m.weight_hash], lr=0.5)
    rng = np.random.default_rng(4)
    for step in range(5):
        ids = torch.from_numpy(zipf_ids(rng, 5000, B))
        w0, h0 = wh.detach().clone(), m.weight_hash.detach().clone()
        out = m(ids)
        rows = m._saved["row"].clone()
        g = torch.randn(B, D, device="cuda")
        opt.zero_grad()
        out.backward(g)
        assert wh.grad.is_sparse and m.weight_hash.grad.is_sparse
        m.insert_grad(ids)
        opt.step()
        hot = rows < 0
        exp_h = w0.clone()
        exp_c = h0.clone()
        # (migration may also have written hot rows; compare only rows the gradient touched and
        # migration did not)
        exp_c.index_add_(0, rows[~hot].long(), -0.5 * g[~hot])
        np.testing.assert_allclose(m.weight_hash.detach().cpu().numpy(), exp_c.cpu().numpy(), rtol=RTOL, atol=1e-6)
        if hot.any():
            exp_h.index_add_(0, (-rows[hot]).long(), -0.5 * g[hot])
            touched = torch.unique((-rows[hot]).long())
            np.testing.assert_allclose(wh.detach()[touched].cpu().numpy(), exp_h[touched].cpu().numpy(), rtol=RTOL, atol=1e-6)


def test_checkpoint_resume_through_state_dict(tmp_path):
    """torch.save(model.state_dict()) carries the sketch; a resumed run continues bit for bit."""
    import torch
    import cafe_b200
    cards, D, B = [5000, 120000, 800000], 16, 128
    rng = np.random.default_rng(8)
    a = cafe_b200.SKEmbeddingGroup(cards, D, 0.01, 0.3, 1, 1, 1.0000005, device="cuda", max_batch=B, lr=0.1, seed=1)
    batches = [np.stack([zipf_ids(rng, n, B) for n in cards]) for _ in range(12)]
    grads = [torch.from_numpy((rng.standard_normal((B, 3, D)) * 0.01).astype(np.float32)).cuda() for _ in range(12)]
    for s in range(6):
        a(torch.from_numpy(batches[s])).backward(grads[s])
    torch.save(a.state_dict(), tmp_path / "ckpt.pt")
    b = cafe_b200.SKEmbeddingGroup(cards, D, 0.01, 0.3, 1, 1, 1.0000005, device="cuda", max_batch=B, lr=0.1, seed=99)
    b.load_state_dict(torch.load(tmp_path / "ckpt.pt", weights_only=False))
    for s in range(6, 12):
        oa = a(torch.from_numpy(batches[s]))
        ob = b(torch.from_numpy(batches[s]))
        assert torch.equal(oa, ob)
        oa.backward(grads[s])
        ob.backward(grads[s])
    assert states_equal(a.sketch.state(), b.sketch.state()) == []
    assert torch.equal(a.weight_high, b.weight_high)
    for wa, wb in zip(a.weight_hash, b.weight_hash):
        assert torch.equal(wa, wb)


def test_backward_head_start_is_only_a_head_start():
    """The sorts started at forward time (training mode) must not change any result: interleaved
    forwards and backwards, where the head start belongs to another batch than the backward that
    follows, give the same bits as a module that never takes the head start (eval mode)."""
    import torch
    import cafe_b200
    cards = [4000, 150000, 61, 700000]
    F, D, B = len(cards), 32, 192
    mk = lambda: cafe_b200.SKEmbeddingGroup(cards, D, 0.01, 0.3, 1, 1, 1.0000005, device="cuda", max_batch=B, lr=0.1, seed=3)
    a, b = mk(), mk()
    b.eval()                                   # no head start; the backward does all the work itself
    rng = np.random.default_rng(11)
    for step in range(6):
        idsA = torch.from_numpy(np.stack([zipf_ids(rng, n, B) for n in cards]))
        idsB = torch.from_numpy(np.stack([zipf_ids(rng, n, B) for n in cards]))
        gA = torch.from_numpy((rng.standard_normal((B, F, D)) * 0.01).astype(np.float32)).cuda()
        gB = torch.from_numpy((rng.standard_normal((B, F, D)) * 0.01).astype(np.float32)).cuda()
        for m in (a, b):
            oA = m(idsA)
            oB = m(idsB)                       # the head start now belongs to batch B ...
            oA.backward(gA)                    # ... and this backward must notice that
            oB.backward(gB)
            if step % 2:
                m(idsA).backward(gA)           # the plain case: head start used by its own backward
        assert states_equal(a.sketch.state(), b.sketch.state()) == [], f"step {step}: sketch state"
        assert torch.equal(a.weight_high, b.weight_high), f"step {step}: hot table"
        for f in range(F):
            assert torch.equal(a.weight_hash[f], b.weight_hash[f]), f"step {step}: hash table {f}"


def test_gated_backward_waits_for_late_fields():
    """cafe_embed_backward_gated: the gradient rows of the later fields are written by another stream, well
    after the call has been made; the result must be the ordinary backward's, bit for bit."""
    import torch
    import cafe_b200
    cards = [4000, 150000, 61, 700000, 2500, 90000]
    F, D, B = len(cards), 32, 1024
    mk = lambda: cafe_b200.SKEmbeddingGroup(cards, D, 0.01, 0.3, 1, 1, 1.0000005, device="cuda", max_batch=B, lr=0.1, seed=9)
    a, b = mk(), mk()
    a.eval(); b.eval()                          # no head start: the calls below drive the field set directly
    rng = np.random.default_rng(21)
    side = torch.cuda.Stream()
    for step in range(8):
        ids = torch.from_numpy(np.stack([zipf_ids(rng, n, B) for n in cards])).cuda()
        g = torch.from_numpy((rng.standard_normal((B, F, D)) * 0.01).astype(np.float32)).cuda()
        flat = ids.reshape(-1)
        outs = []
        for m in (a, b):
            out = torch.empty(B, F, D, dtype=torch.float32, device="cuda")
            gid, row = m._fields.forward(flat, out, D, F * D)
            outs.append((gid, row))
        b._fields.backward(g, D, F * D, flat, outs[1][0], outs[1][1], B, b.lr, b.insert_mode)
        gate = 1 + step % (F - 1)
        late = torch.full_like(g, float("nan"))             # what the backward must not read too early
        late[:, :gate] = g[:, :gate]
        ev = torch.cuda.Event()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            torch.cuda._sleep(3_000_000)                    # about 1.5 ms: the gated call is queued long before
            late[:, gate:] = g[:, gate:]
            ev.record(side)
        a._fields.backward_gated(late, D, F * D, flat, outs[0][0], outs[0][1], B, a.lr, a.insert_mode, gate, ev)
        torch.cuda.synchronize()
        assert states_equal(a.sketch.state(), b.sketch.state()) == [], f"step {step}: sketch state"
        assert torch.equal(a.weight_high, b.weight_high), f"step {step}: hot table"
        for f in range(F):
            assert torch.equal(a.weight_hash[f], b.weight_hash[f]), f"step {step}: hash table {f}"


def test_two_fields_claim_one_hot_row_in_one_step():
    """A threshold re-fit between two fields' calls of one step takes a hot row from an id of the earlier field and an
    id of the later field pops it: both lookups are reported newly hot with the same row.  The reference migrates
    field by field, so the later field's hash row is the one that stays in the hot table (the configuration below
    reaches this case within its 30 steps with the sequential oracle)."""
    import torch
    import cafe_b200
    F, B, dom, D, lim = 8, 128, 2000, 16, 60
    cards = [dom] * F
    grp = cafe_b200.SKEmbeddingGroup(cards, D, 0.01, 0.3, 1, 1, 1.0000005, device="cuda", max_batch=B, lr=0.1, seed=3, hotn=lim)
    sk = OracleSketch(lim, 1, 1, 1.0000005)
    orc = ModuleOracle(sk, grp.weight_high.detach().cpu().numpy(), [w.detach().cpu().numpy() for w in grp.weight_hash],
                       grp.f_offsets, grp.hash_sizes)
    rng = np.random.default_rng(0)
    for step in range(30):
        ids = np.stack([np.minimum(rng.zipf(1.2, B) - 1, dom - 1) for _ in range(F)]).astype(np.int64)
        imp = (rng.random((F, B)) * 2).astype(np.float32)
        # gradient rows whose norms are the wanted importances times a constant: both sides get the kernel's floats
        grad = np.zeros((B, F, D), np.float32)
        grad[:, :, 0] = imp.T * 0.01
        out = grp(torch.from_numpy(ids))
        orc.forward(ids)
        g = torch.from_numpy(grad).cuda()
        impk = grp._fields.importance(g, D, F * D, B).view(F, B).cpu().numpy()
        out.backward(g)
        masks, _ = orc.backward(ids, grad, grp.lr, importance=impk)
        assert states_equal(sk.state(), grp.sketch.state()) == [], f"step {step}"
        close(grp.weight_high.detach().cpu().numpy(), orc.wh, f"step {step}: hot table")
    assert grp.sketch.stats()["resets"] > 0
