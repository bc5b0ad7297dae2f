"""Field-sharding index arithmetic on CPU: 2 and 3 gloo ranks exchange ids, pooled rows and gradients
with the same code the NCCL path uses, and the result is compared with a single-process computation."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cafe_b200.sharded import FieldShardPlan


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def fake_embed(field, ids, D):
    """Deterministic stand-in for a table lookup: row depends on (field, id)."""
    base = (ids.double() * 0.001 + field * 7.0)[..., None]
    return (base + torch.arange(D).double() * 0.5).float()


def _worker(rank, world, port, F, Bl, D, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        plan = FieldShardPlan(F, world, rank)
        g = torch.Generator().manual_seed(100 + rank)
        ids = torch.randint(0, 10_000, (F, Bl), generator=g)
        own = plan.exchange_ids(ids)
        Fg = len(plan.local_fields)
        assert own.shape == (Fg, world * Bl)
        # owners compute their fields for the global batch: [B_global, F_g, D]
        pooled = torch.stack([fake_embed(f, own[j], D) for j, f in enumerate(plan.local_fields)], dim=1) if Fg else \
            torch.empty(world * Bl, 0, D)
        blocked = plan.exchange_pooled(pooled.contiguous())
        full = plan.unblock(blocked, Bl, D)
        want = torch.stack([fake_embed(f, ids[f], D) for f in range(F)], dim=1)
        ok_fwd = torch.equal(full, want)
        ok_rt = torch.equal(plan.block(full), blocked)
        # gradients: each rank sends grad of its [B_local, F, D]; owners must receive [B_global, F_g, D]
        grad_full = want * (rank + 1)
        got = plan.exchange_grads(plan.block(grad_full), Bl, D)
        # what every rank sent, recomputed locally from the gathered ids
        exp = torch.stack([fake_embed(f, own[j], D) for j, f in enumerate(plan.local_fields)], dim=1) if Fg else got
        scale = torch.arange(1, world + 1).repeat_interleave(Bl).float()[:, None, None]
        ok_bwd = torch.equal(got, exp * scale) if Fg else True
        q.put((rank, ok_fwd, ok_rt, ok_bwd))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,F", [(2, 5), (3, 7), (2, 26)])
def test_exchanges_match_single_process(world, F):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, F, 6, 4, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert all(ok_f and ok_r and ok_b for _, ok_f, ok_r, ok_b in res), res


def test_plan_covers_every_field_once():
    for world in (1, 2, 4, 8):
        plans = [FieldShardPlan(26, world, r) for r in range(world)]
        seen = sorted(f for p in plans for f in p.local_fields)
        assert seen == list(range(26))
        assert sorted(plans[0].blocked_order) == list(range(26))
        assert max(plans[0].counts) - min(plans[0].counts) <= 1


def _subgroup_worker(rank, world, port, members, F, Bl, D, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sub = dist.new_group(ranks=members)   # every rank takes part in creating it
        if rank not in members:
            q.put((rank, True, True))
            return
        G, r = len(members), members.index(rank)
        plan = FieldShardPlan(F, G, r)
        g = torch.Generator().manual_seed(100 + r)
        ids = torch.randint(0, 10_000, (F, Bl), generator=g)
        own = plan.exchange_ids(ids, sub)
        Fg = len(plan.local_fields)
        pooled = torch.stack([fake_embed(f, own[j], D) for j, f in enumerate(plan.local_fields)], dim=1)
        full = plan.unblock(plan.exchange_pooled(pooled.contiguous(), sub), Bl, D)
        want = torch.stack([fake_embed(f, ids[f], D) for f in range(F)], dim=1)
        got = plan.exchange_grads(plan.block(want * (r + 1)), Bl, D, sub)
        scale = torch.arange(1, G + 1).repeat_interleave(Bl).float()[:, None, None]
        q.put((rank, torch.equal(full, want), torch.equal(got, pooled * scale)))
    finally:
        dist.destroy_process_group()


def test_exchanges_on_a_subgroup_of_the_job():
    """Fields sharded over ranks 1 and 3 of a four-rank job: the exchanges run on that group only, and the other
    ranks are not needed for them to finish."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_subgroup_worker, args=(r, 4, port, [1, 3], 7, 5, 4, q)) for r in range(4)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(4)]
    for p in procs:
        p.join(timeout=60)
    assert all(a and b for _, a, b in res), res


def test_shard_capacity_by_fields_and_by_rows():
    """Terabyte cardinalities at compress 1e-4 / hash-rate 0.2 / dim 128 over 8 ranks, fields round-robin: sized from
    its own rows, the rank that owns fields 7, 15 and 23 (1 543 + 155 + 12 972 ids) would get a capacity of 1 (the
    reference's constructor divides by int(0.1 * lim) = 0); sized by field count every rank gets 3/26 or 4/26 of the
    13 733 rows the reference's formula gives for all fields."""
    from cafe_b200 import sizing
    from cafe_b200.synthetic import TERABYTE_CARDS
    cards = list(TERABYTE_CARDS)
    total = sizing.hot_rows(sum(cards), 1e-4, 0.2, 128)
    assert total == 13733
    shares = []
    for r in range(8):
        mine = list(range(r, 26, 8))
        shares.append(sizing.shard_hot_rows(cards, mine, 1e-4, 0.2, 128, "fields"))
        assert shares[-1] == total * len(mine) // 26
    assert sum(shares) <= total and min(shares) >= 1584
    assert sizing.hot_rows(sum(cards[f] for f in (7, 15, 23)), 1e-4, 0.2, 128) == 1
    assert sizing.shard_hot_rows(cards, [7, 15, 23], 1e-4, 0.2, 128, "rows") == 20


class _ReplicatedTables(torch.nn.Module):
    """CPU stand-in for the embedding layer of the DLRM harness: one dense table per field on every rank."""

    def __init__(self, cards, D):
        super().__init__()
        g = torch.Generator().manual_seed(9)
        self.tables = torch.nn.ParameterList([torch.nn.Parameter(torch.randn(n, D, generator=g) * 0.1) for n in cards])
        self.device = torch.device("cpu")
        self.group = None

    def set_lr(self, lr):
        pass

    def forward(self, lS_o, lS_i, test=False):
        # the last table is looked up with a sparse gradient, as the small plain tables of the sharded layer are
        cols = [t[i] for t, i in zip(self.tables[:-1], lS_i)]
        cols.append(torch.nn.functional.embedding(lS_i[-1], self.tables[-1], sparse=True))
        return torch.stack(cols, dim=1)


def _dlrm_batches(cards, B, steps):
    g = torch.Generator().manual_seed(77)
    out = []
    for _ in range(steps):
        ids = torch.stack([torch.randint(0, n, (B,), generator=g) for n in cards])
        out.append((torch.randn(B, 5, generator=g), ids, (torch.rand(B, generator=g) < 0.3).float()))
    return out


def _dlrm_model(cards, D):
    from cafe_b200 import dlrm_harness as H
    return H.DLRMNet(cards, D, [5, 16, D], [16, 1], _ReplicatedTables(cards, D), seed=3)


def _dp_worker(rank, world, port, cards, D, Bl, steps, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cafe_b200 import dlrm_harness as H
        torch.set_num_threads(1)
        model = _dlrm_model(cards, D)
        opt = torch.optim.SGD(H.dense_and_plain_parameters(model), lr=0.5)
        shares = []
        for dense, ids, y in _dlrm_batches(cards, Bl * world, steps):
            sl = slice(rank * Bl, (rank + 1) * Bl)
            loss, _ = H.train_step_data_parallel(model, opt, dense[sl], None, ids[:, sl], y[sl])
            shares.append(float(loss.detach()))
        q.put((rank, shares, [p.detach().numpy().copy() for p in model.parameters()]))
    finally:
        dist.destroy_process_group()


def test_data_parallel_step_equals_one_process_on_the_global_batch():
    """Two ranks, each with half of every batch, against one process fed the whole batch: the ranks' loss shares add
    up to the global loss and after three steps every parameter (MLPs and tables) agrees within fp32 rounding."""
    from cafe_b200 import dlrm_harness as H
    cards, D, Bl, steps, world = [50, 7, 300], 8, 12, 3, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_dp_worker, args=(r, world, port, cards, D, Bl, steps, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=120) for _ in range(world)], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
    model = _dlrm_model(cards, D)
    opt = torch.optim.SGD(H.dense_and_plain_parameters(model), lr=0.5)
    losses = []
    for dense, ids, y in _dlrm_batches(cards, Bl * world, steps):
        loss, _ = H.train_step(model, opt, dense, None, ids, y)
        losses.append(float(loss.detach()))
    for s in range(steps):
        assert abs(sum(r[1][s] for r in res) - losses[s]) < 1e-6
    for r in res:
        for a, b in zip(r[2], model.parameters()):
            assert torch.allclose(torch.from_numpy(a), b.detach(), rtol=1e-5, atol=1e-7)
    for a, b in zip(res[0][2], res[1][2]):
        assert (a == b).all()
