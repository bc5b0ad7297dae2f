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

Two ways to do the exchange: `exchange="nccl"` (library all-to-all, the baseline) and `exchange="peer"`
(default): buffers live in symmetric memory mapped into every rank, the gather kernel stores each pooled
row straight into the consuming rank's buffer, and the owner pulls gradient rows from the consumers while
it computes their norms (cafe_embed_forward_sharded / cafe_shard_pull_importance), so the transfers
overlap the kernels' own work row by row; ranks are ordered by three one-element all-reduces per step.
"""
from __future__ import annotations

import ctypes
import os

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


class PeerBuffers:
    """Symmetric-memory buffers of one rank and the addresses of every rank's copies.

    ids    [2][Fmax * G * B_local] int64 : this rank as OWNER: ids of its fields for the global batch
                                           (two generations, so that a fast peer never overwrites ids
                                           the owner is still reading in its backward)
    pooled [B_local * F * D] fp32        : this rank as CONSUMER: pooled rows of its batch slice, blocks
                                           [B_local, F_r, D] ordered by owner r
    grad   [B_local * F * D] fp32        : this rank as CONSUMER: gradient of `pooled`, same layout
    gown   [G * B_local * Fmax * D] fp32 : this rank as OWNER: gradient rows of its fields for the global
                                           batch, stored there by the consumers
    """

    def __init__(self, plan: "FieldShardPlan", rows: int, dim: int, device, group=None):
        # plain peer mappings only: no NVLink multicast objects are bound to these buffers
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        grp = group if group is not None else dist.group.WORLD
        self.plan, self.rows, self.dim, self.pg = plan, rows, dim, group
        fmax = max(plan.counts)
        self.ids = symm.empty(2 * fmax * plan.G * rows, dtype=torch.int64, device=device)
        self.pooled = symm.empty(rows * plan.F * dim, dtype=torch.float32, device=device)
        self.grad = symm.empty(rows * plan.F * dim, dtype=torch.float32, device=device)
        self.gown = symm.empty(plan.G * rows * fmax * dim, dtype=torch.float32, device=device)   # as OWNER: gradients of its fields, global batch
        self.nown = symm.empty(fmax * plan.G * rows, dtype=torch.float32, device=device)         # as OWNER: their L2 norms [F_g, B]
        self.h_ids = symm.rendezvous(self.ids, grp)
        self.h_pooled = symm.rendezvous(self.pooled, grp)
        self.h_grad = symm.rendezvous(self.grad, grp)
        self.h_gown = symm.rendezvous(self.gown, grp)
        self.h_nown = symm.rendezvous(self.nown, grp)
        self.ids_gen_elems = fmax * plan.G * rows
        # offset (elements) of owner r's block inside every consumer's pooled / grad buffer
        self.block_off = [rows * dim * sum(plan.counts[:r]) for r in range(plan.G)]
        self.nsend = torch.empty(rows * plan.F, dtype=torch.float32, device=device)   # norms of this rank's rows, staged
        self.flag = torch.zeros(1, device=device)
        self.gen = 0
        with torch.cuda.device(device):
            self.comm_stream = torch.cuda.Stream()        # the gradient exchange when it is issued in pieces
            self.ev_first, self.ev_second, self.ev_grad = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()

    def ptr_array(self, handle, elem_offset: int, elem_size: int):
        return (ctypes.c_void_p * self.plan.G)(*[int(p) + elem_offset * elem_size for p in handle.buffer_ptrs])

    def fence(self):
        """All ranks of the group have issued everything before this point on their streams (stream-ordered)."""
        dist.all_reduce(self.flag, group=self.pg)


class _PeerFunction(torch.autograd.Function):
    """The exchange folded into the kernels (see the module docstring)."""

    @staticmethod
    def forward(ctx, anchor, model, ids):
        from . import _lib
        from .sketch import _stream
        plan, grp, pb = model.plan, model.group, model.peer
        lib = grp.sketch.lib
        F, Bl = ids.shape
        G, Fg, D = plan.G, grp.num_fields, grp.embedding_dim
        training = bool(ctx.needs_input_grad[0])
        if training and model._pending_backward:
            raise RuntimeError("ShardedSKEmbedding (peer exchange): a second training forward before the backward of the "
                               "previous one would overwrite the exchange buffers that backward still reads")
        pb.gen ^= 1
        gen_off = pb.gen * pb.ids_gen_elems
        with torch.cuda.device(ids.device):
            _lib.check(lib.cafe_shard_scatter_ids(ids.data_ptr(), F, Bl, G, plan.rank, pb.ptr_array(pb.h_ids, gen_off, 8),
                                                  _stream()), "cafe_shard_scatter_ids")
            pb.fence()                                   # every owner now holds the global batch's ids
            own = pb.ids[gen_off:gen_off + Fg * G * Bl]  # [F_g, G*B_local], field-major
            gid = torch.empty(own.numel(), dtype=torch.int32, device=ids.device)
            row = torch.empty(own.numel(), dtype=torch.int32, device=ids.device)
            f = grp._fields
            wp, hp = f.ptrs()
            out_rank = pb.ptr_array(pb.h_pooled, pb.block_off[plan.rank], 4)
            if training:
                # sketch probe, then the backward's sorts on the side streams, then the gather with the exchange as
                # its epilogue: the sorts run beside the gather and the dense model
                _lib.check(lib.cafe_embed_resolve(grp.sketch.handle, own.data_ptr(), 1, Fg, G * Bl, f.f_offset, f.hash_size,
                                                  f.hotn, gid.data_ptr(), row.data_ptr(), _stream()), "cafe_embed_resolve")
                f.backward_begin(gid, row, G * Bl, grp.insert_mode)
                _lib.check(lib.cafe_embed_gather_sharded(grp.sketch.handle, row.data_ptr(), Fg, G * Bl, f.hash_size, wp, hp,
                                                         f.hotn, D, out_rank, G, Bl, D, Fg * D, _stream()),
                           "cafe_embed_gather_sharded")
            else:
                _lib.check(lib.cafe_embed_forward_sharded(grp.sketch.handle, own.data_ptr(), 1, Fg, G * Bl, f.f_offset,
                                                          f.hash_size, wp, hp, f.hotn, D, out_rank, G, Bl, D, Fg * D,
                                                          gid.data_ptr(), row.data_ptr(), _stream()),
                           "cafe_embed_forward_sharded")
            pb.fence()                                   # every consumer's pooled buffer is complete
        ctx.model, ctx.saved, ctx.Bl = model, (own, gid, row), Bl
        model._pending_backward = training
        return pb.pooled

    @staticmethod
    def backward(ctx, blocked_grad):
        from . import _lib
        from .sketch import _stream
        model = ctx.model
        model._pending_backward = False
        plan, grp, pb = model.plan, model.group, model.peer
        lib = grp.sketch.lib
        own, gid, row = ctx.saved
        G, Fg, D, Bl = plan.G, grp.num_fields, grp.embedding_dim, ctx.Bl
        f = grp._fields
        with torch.no_grad(), torch.cuda.device(pb.grad.device):
            g = blocked_grad.reshape(-1).contiguous()   # (the backward's sorts were started by the forward)
            half = (plan.F // G) // 2     # same on every rank: owners' fields 0..half-1 travel first
            if model.push == "norms_first" and G > 1:
                # The rows' L2 norms (4 bytes per lookup) go first; with them the owners run importance and the whole
                # sketch insert while the rows themselves cross NVLink on a stream of their own.  Only the SGD scatter
                # reads the rows, and only it waits for them.
                main, comm = torch.cuda.current_stream(), pb.comm_stream
                _lib.check(lib.cafe_shard_push_norms(g.data_ptr(), plan.F, Bl, D, G, plan.rank,
                                                     pb.ptr_array(pb.h_nown, 0, 4), pb.nsend.data_ptr(), _stream()),
                           "cafe_shard_push_norms")
                pb.ev_grad.record(main)                     # (the rows start once the norms have left)
                pb.fence()                                  # every owner holds the norms of the global batch
                comm.wait_event(pb.ev_grad)
                g.record_stream(comm)
                with torch.cuda.stream(comm):
                    _lib.check(lib.cafe_shard_push_grads(g.data_ptr(), plan.F, Bl, D, G, plan.rank,
                                                         pb.ptr_array(pb.h_gown, 0, 4), comm.cuda_stream), "cafe_shard_push_grads")
                    pb.fence()                              # every owner holds the rows (issued second on every rank)
                    pb.ev_second.record(comm)
                grp.last_status = f.backward_norms(pb.gown, D, Fg * D, pb.nown, own, gid, row, G * Bl, grp.lr, grp.insert_mode,
                                                   pb.ev_second)
            elif not model.pipeline_push or G == 1 or half < 1:
                # consumers store their gradient rows into the owners' buffers (remote stores over NVLink) ...
                _lib.check(lib.cafe_shard_push_grads(g.data_ptr(), plan.F, Bl, D, G, plan.rank,
                                                     pb.ptr_array(pb.h_gown, 0, 4), _stream()), "cafe_shard_push_grads")
                pb.fence()
                # ... and every owner runs the ordinary fused backward on its local buffer [G*B_local, F_g, D]
                grp.last_status = f.backward(pb.gown, D, Fg * D, own, gid, row, G * Bl, grp.lr, grp.insert_mode)
            else:
                # The same in two pieces on a stream of its own: while the second piece crosses NVLink, the
                # owners already compute the importance of the first piece's fields and insert them (the
                # insert takes the fields in ascending order anyway); the gated backward waits for the
                # second piece only when it gets to its fields.
                main, comm = torch.cuda.current_stream(), pb.comm_stream
                comm.wait_stream(main)
                g.record_stream(comm)
                owners = pb.ptr_array(pb.h_gown, 0, 4)
                with torch.cuda.stream(comm):
                    _lib.check(lib.cafe_shard_push_grads_fields(g.data_ptr(), plan.F, Bl, D, G, plan.rank, owners, 0, half,
                                                                comm.cuda_stream), "cafe_shard_push_grads_fields")
                    pb.fence()
                    pb.ev_first.record(comm)
                    _lib.check(lib.cafe_shard_push_grads_fields(g.data_ptr(), plan.F, Bl, D, G, plan.rank, owners, half,
                                                                1 << 30, comm.cuda_stream), "cafe_shard_push_grads_fields")
                    pb.fence()
                    pb.ev_second.record(comm)
                main.wait_event(pb.ev_first)
                grp.last_status = f.backward_gated(pb.gown, D, Fg * D, own, gid, row, G * Bl, grp.lr, grp.insert_mode,
                                                   half, pb.ev_second)
        return None, None, None


class _ShardedFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, anchor, model, ids):
        plan, grp = model.plan, model.group
        Bl = ids.shape[1]
        own_ids = plan.exchange_ids(ids, model.pg)
        flat = own_ids.reshape(-1)
        Fg, D = grp.num_fields, grp.embedding_dim
        pooled = torch.empty(plan.G * Bl, Fg, D, dtype=torch.float32, device=ids.device)
        if ctx.needs_input_grad[0] and flat.numel() > 0:
            gid, row = grp._fields.forward_training(flat, pooled, D, Fg * D, grp.insert_mode)   # starts the backward's sorts
        else:
            gid, row = grp._fields.forward(flat, pooled, D, Fg * D)
        ctx.model, ctx.saved, ctx.Bl = model, (flat, gid, row), Bl
        return plan.exchange_pooled(pooled, model.pg)

    @staticmethod
    def backward(ctx, blocked_grad):
        model = ctx.model
        plan, grp = model.plan, model.group
        flat, gid, row = ctx.saved
        Fg, D = grp.num_fields, grp.embedding_dim
        g = plan.exchange_grads(blocked_grad.contiguous(), ctx.Bl, D, model.pg)
        with torch.no_grad():
            grp.last_status = grp._fields.backward(g, D, Fg * D, flat, gid, row, plan.G * ctx.Bl, grp.lr, grp.insert_mode)
        return None, None, None


class ShardedSKEmbedding(torch.nn.Module):
    """forward(ids [F, B_local]) -> rank-blocked pooled embeddings of this rank's batch slice
    (see FieldShardPlan.unblock for the [B_local, F, D] view); backward runs the fused update on the
    owners.  Needs an initialised NCCL process group with one rank per GPU; `group` (default: all ranks)
    is the set of ranks the fields are sharded over, and every exchange and fence runs on it.

    With the peer exchange the tensor a training forward returns IS this rank's exchange buffer: it is valid
    until the next forward() of this module, whose peers overwrite it by remote stores that autograd does not
    see.  Therefore a second forward before the backward of a training forward raises (gradient accumulation
    over several forwards and evaluation between a forward and its backward are not supported); a forward
    under no_grad, between steps, returns a copy."""

    def __init__(self, num_categories, embedding_dim, compress_rate, hash_rate, sketch_threshold=1, adjust_threshold=1,
                 sketch_alpha=1.0000005, device="cuda", global_batch=65536, lr=0.1, seed=None, group=None,
                 exchange="peer", f_offsets=None, pipeline_push=False, hot_rows_by="fields", push="norms_first"):
        super().__init__()
        from .sk_embedding_bag import SKEmbeddingGroup
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        if rank < 0:
            raise ValueError("this rank is not a member of `group`")
        self.pg = group
        self._pending_backward = False
        cards = [int(n) for n in num_categories]
        self.num_categories = cards
        self.plan = FieldShardPlan(len(cards), world, rank)
        # global ids (id + offset) must stay below 2**31; with very many fields pass offsets that are only
        # distinct within each rank (ranks never share sketch state)
        offs = list(f_offsets) if f_offsets is not None else sizing.field_offsets(cards)
        if max(o + n for o, n in zip(offs, cards)) > 2 ** 31:
            raise ValueError("field offsets push ids beyond 2**31; pass per-rank offsets via f_offsets")
        mine = self.plan.local_fields
        if not mine:
            raise ValueError("more ranks than fields")
        self.embedding_dim = int(embedding_dim)
        self.global_batch = int(global_batch)
        hotn = sizing.shard_hot_rows(cards, mine, compress_rate, hash_rate, self.embedding_dim, hot_rows_by)
        self.group = SKEmbeddingGroup([cards[f] for f in mine], embedding_dim, compress_rate, hash_rate, sketch_threshold,
                                      adjust_threshold, sketch_alpha, device=device, max_batch=global_batch, lr=lr,
                                      f_offsets=[offs[f] for f in mine], hotn=hotn,
                                      seed=None if seed is None else seed + rank)
        self._anchor = torch.nn.Parameter(torch.zeros(1, device=self.group.weight_high.device))
        self.h2d_bytes = self.d2h_bytes = 0
        if exchange not in ("peer", "nccl"):
            raise ValueError("exchange must be 'peer' or 'nccl'")
        self.exchange = exchange
        # gradient exchange in two pieces, the second beside the first piece's insert.  Off by default: on two GPUs
        # the job boundary it forces at the gate cost more than the hidden half of the transfer gave back.
        self.pipeline_push = bool(pipeline_push)
        # "norms_first": the rows' norms travel ahead and the sketch insert runs beside the rows' transfer; "whole":
        # rows first, then the ordinary backward (pipeline_push=True splits that into two pieces)
        if push not in ("norms_first", "whole"):
            raise ValueError("push must be 'norms_first' or 'whole'")
        self.push = "whole" if self.pipeline_push else push
        self.peer = None
        self._gbuf = self._imp = None
        if exchange == "peer":
            if world > 8:
                raise ValueError("the peer-memory exchange serves one node (at most 8 ranks)")
            self.peer = PeerBuffers(self.plan, self.global_batch // world, self.embedding_dim,
                                    self.group.weight_high.device, group)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        ids = ids.to(self.group.weight_high.device, non_blocking=True).contiguous()
        if self.peer is not None:
            if ids.dtype != torch.int64 or ids.shape[1] != self.peer.rows:
                raise ValueError("peer exchange: ids must be int64 [F, global_batch / world]")
            if not torch.is_grad_enabled():
                if self._pending_backward:
                    raise RuntimeError("ShardedSKEmbedding (peer exchange): forward under no_grad between a training "
                                       "forward and its backward would overwrite the buffers that backward reads")
                return _PeerFunction.apply(self._anchor, self, ids).clone()
            return _PeerFunction.apply(self._anchor, self, ids)
        return _ShardedFunction.apply(self._anchor, self, ids)
