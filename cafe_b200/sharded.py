"""Field-sharded CAFE embeddings across the GPUs of one node.

The reference is single-GPU (its --dist flags are parsed and never used, dlrm_s_pytorch.py:1090-1091);
this module adds the one parallelism the hot path admits: every rank owns a subset of the sketch
fields (round robin), with its own hash tables, hot table and sketch, and serves the GLOBAL batch for
those fields.  Per step there is one exchange each way:

  ids      [F, B_local] per rank   --all-to-all-->  [F_g, B_global] on the owner of the fields
  pooled   [B_global, F_g, D]      --all-to-all-->  blocks [B_local, F_r, D] from every owner r
  grads    the transpose of the pooled exchange; they arrive on the owner as [B_global, F_g, D],
           exactly the layout the fused backward reads.

Each shard is bit-identical to an independent single-GPU run over its own fields with the global
field offsets (there is no cross-rank state).  `FieldShardPlan` and the exchange functions are plain
torch.distributed code and also run on CPU tensors under the gloo backend, which is how the index
arithmetic is tested without GPUs.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import sizing


class FieldShardPlan:
    """Which rank owns which field, and the split sizes of the exchanges."""

    def __init__(self, num_fields: int, world: int, rank: int):
        self.F, self.G, self.rank = int(num_fields), int(world), int(rank)
        self.owner = [f % self.G for f in range(self.F)]
        self.fields_of = [[f for f in range(self.F) if f % self.G == r] for r in range(self.G)]
        self.local_fields = self.fields_of[self.rank]
        self.counts = [len(x) for x in self.fields_of]
        # position of global field f inside the rank-blocked layout (owner-major, then local order)
        self.blocked_order = [f for r in range(self.G) for f in self.fields_of[r]]

    # ---- ids: [F, B_local] on every rank -> [F_g, G*B_local] on owners ---------------------------
    def exchange_ids(self, ids: torch.Tensor, group=None) -> torch.Tensor:
        F, Bl = ids.shape
        assert F == self.F
        send = ids[self.blocked_order].contiguous()            # owner-major rows
        in_split = [c * Bl for c in self.counts]
        Fg = self.counts[self.rank]
        recv = torch.empty(self.G * Fg * Bl, dtype=ids.dtype, device=ids.device)
        dist.all_to_all_single(recv, send.view(-1), [Fg * Bl] * self.G, in_split, group=group)
        # recv is [G (source rank = batch slice), F_g, B_local] -> [F_g, G, B_local] -> [F_g, B_global]
        return recv.view(self.G, Fg, Bl).permute(1, 0, 2).reshape(Fg, self.G * Bl).contiguous()

    # ---- pooled: [B_global, F_g, D] on owners -> rank-blocked [sum_r B_local*F_r*D] -------------
    def exchange_pooled(self, pooled: torch.Tensor, group=None) -> torch.Tensor:
        Bg, Fg, D = pooled.shape
        Bl = Bg // self.G
        out_split = [Bl * c * D for c in self.counts]
        recv = torch.empty(sum(out_split), dtype=pooled.dtype, device=pooled.device)
        dist.all_to_all_single(recv, pooled.reshape(-1), out_split, [Bl * Fg * D] * self.G, group=group)
        return recv

    # ---- grads: rank-blocked gradient of the pooled exchange -> [B_global, F_g, D] on owners -------
    def exchange_grads(self, blocked_grad: torch.Tensor, Bl: int, D: int, group=None) -> torch.Tensor:
        Fg = self.counts[self.rank]
        in_split = [Bl * c * D for c in self.counts]
        recv = torch.empty(self.G * Bl * Fg * D, dtype=blocked_grad.dtype, device=blocked_grad.device)
        dist.all_to_all_single(recv, blocked_grad.reshape(-1), [Bl * Fg * D] * self.G, in_split, group=group)
        return recv.view(self.G * Bl, Fg, D)

    # ---- layout helpers -----------------------------------------------------------------------------
    def blocks(self, blocked: torch.Tensor, Bl: int, D: int):
        """Views [B_local, F_r, D] of the rank-blocked buffer, one per owner r."""
        out, o = [], 0
        for c in self.counts:
            n = Bl * c * D
            out.append(blocked[o:o + n].view(Bl, c, D))
            o += n
        return out

    def unblock(self, blocked: torch.Tensor, Bl: int, D: int) -> torch.Tensor:
        """[B_local, F, D] in global field order (one strided copy; consumers that can read the
        blocked layout should skip it)."""
        out = torch.empty(Bl, self.F, D, dtype=blocked.dtype, device=blocked.device)
        for r, blk in enumerate(self.blocks(blocked, Bl, D)):
            if blk.shape[1]:
                out[:, r::self.G, :] = blk
        return out

    def block(self, full: torch.Tensor) -> torch.Tensor:
        """Inverse of unblock: [B_local, F, D] -> rank-blocked flat buffer."""
        return torch.cat([full[:, r::self.G, :].reshape(-1) for r in range(self.G)])


class _ShardedFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, anchor, model, ids):
        plan, grp = model.plan, model.group
        Bl = ids.shape[1]
        own_ids = plan.exchange_ids(ids)
        flat = own_ids.reshape(-1)
        Fg, D = grp.num_fields, grp.embedding_dim
        pooled = torch.empty(plan.G * Bl, Fg, D, dtype=torch.float32, device=ids.device)
        gid, row = grp._fields.forward(flat, pooled, D, Fg * D)
        ctx.model, ctx.saved, ctx.Bl = model, (flat, gid, row), Bl
        return plan.exchange_pooled(pooled)

    @staticmethod
    def backward(ctx, blocked_grad):
        model = ctx.model
        plan, grp = model.plan, model.group
        flat, gid, row = ctx.saved
        Fg, D = grp.num_fields, grp.embedding_dim
        g = plan.exchange_grads(blocked_grad.contiguous(), ctx.Bl, D)
        with torch.no_grad():
            grp.last_status = grp._fields.backward(g, D, Fg * D, flat, gid, row, plan.G * ctx.Bl, grp.lr, grp.insert_mode)
        return None, None, None


class ShardedSKEmbedding(torch.nn.Module):
    """forward(ids [F, B_local]) -> rank-blocked pooled embeddings of this rank's batch slice
    (see FieldShardPlan.unblock for the [B_local, F, D] view); backward runs the fused update on the
    owners.  Needs an initialised NCCL process group with one rank per GPU."""

    def __init__(self, num_categories, embedding_dim, compress_rate, hash_rate, sketch_threshold=1, adjust_threshold=1,
                 sketch_alpha=1.0000005, device="cuda", global_batch=65536, lr=0.1, seed=None, group=None):
        super().__init__()
        from .sk_embedding_bag import SKEmbeddingGroup
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        cards = [int(n) for n in num_categories]
        self.plan = FieldShardPlan(len(cards), world, rank)
        offs = sizing.field_offsets(cards)
        mine = self.plan.local_fields
        if not mine:
            raise ValueError("more ranks than fields")
        self.embedding_dim = int(embedding_dim)
        self.global_batch = int(global_batch)
        self.group = SKEmbeddingGroup([cards[f] for f in mine], embedding_dim, compress_rate, hash_rate, sketch_threshold,
                                      adjust_threshold, sketch_alpha, device=device, max_batch=global_batch, lr=lr,
                                      f_offsets=[offs[f] for f in mine], seed=None if seed is None else seed + rank)
        self._anchor = torch.nn.Parameter(torch.zeros(1, device=self.group.weight_high.device))
        self.h2d_bytes = self.d2h_bytes = 0

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        ids = ids.to(self.group.weight_high.device, non_blocking=True).contiguous()
        return _ShardedFunction.apply(self._anchor, self, ids)

    # ---- benchmark plumbing ---------------------------------------------------------------------------
    def bench_closures(self, S, zipf_s, seed):
        """(step_fn, e2e_fn, ids_per_rank_step) for bench.py: every rank feeds its slice of the global
        batch (all fields), gradients of the exchanged embeddings are synthetic N(0, 0.01)."""
        plan, dev = self.plan, self.group.weight_high.device
        Bl, D, F = self.global_batch // plan.G, self.embedding_dim, plan.F
        cards = None
        nb = 4
        import numpy as np
        from . import synthetic
        cards = synthetic.MICRO_CARDS
        host = [torch.from_numpy(S.batch_ids(cards, Bl, zipf_s, seed + 7919 * plan.rank, s)).pin_memory() for s in range(nb)]
        devi = [h.to(dev) for h in host]
        g = torch.Generator(device=dev).manual_seed(seed + plan.rank)
        grads = [torch.randn(Bl * F * D, device=dev, generator=g) * 0.01 for _ in range(2)]
        stage = torch.empty_like(devi[0])
        res = torch.empty(16 * D, dtype=torch.float32).pin_memory()
        self.h2d_bytes, self.d2h_bytes = host[0].numel() * 8 * plan.G, res.numel() * 4 * plan.G

        def step_fn(s):
            out = self(devi[s % nb])
            out.backward(grads[s % 2])

        def e2e_fn(s):
            stage.copy_(host[s % nb], non_blocking=True)
            out = self(stage)
            out.backward(grads[s % 2])
            res.copy_(out.detach()[:16 * D], non_blocking=True)

        return step_fn, e2e_fn, Bl * F
