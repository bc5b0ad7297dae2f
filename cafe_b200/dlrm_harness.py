"""A DLRM / DCN training harness around the CAFE drop-in, with the reference's flags and step order.

What the reference's model scripts do around the compressed-embedding path (dlrm_s_pytorch.py, dcn.py), kept
thin and with the dense side on stock PyTorch:

  * flags  --sketch-flag --compress-rate --hash-rate --sketch-threshold --adjust-threshold --sketch-alpha
           --notinsert-test with the reference's defaults (dlrm_s_pytorch.py:1017-1020, 1114, 1126-1128);
  * sizing hotn = int(totn * cr * (1 - hr) * (4D / (4D + 48))) over ALL fields, hash rows round(cr*hr*n + 0.51),
           field offsets over all fields (dlrm_s_pytorch.py:1236-1242, 319, 351-353);
  * create_emb's split (dlrm_s_pytorch.py:309-322): fields with n > 2000 * compress_rate go through the sketch
           (here: one SKEmbeddingGroup for all of them), the others keep a plain nn.EmbeddingBag(mode="sum",
           sparse=True) initialised uniform(+-sqrt(1 / max(n, 5)));
  * the model: bottom MLP -> embeddings -> dot interaction -> top MLP with a final sigmoid
           (dlrm_s_pytorch.py:213-251, 779-850), or the DCN head of dcn.py:410-422, 712-742 (cross layers + deep MLP);
  * the step (dlrm_s_pytorch.py:1610-1659): forward, BCE loss, zero_grad, backward, insert_grad, optimizer.step.
           With SKEmbeddingGroup the importance -> insert -> migration -> SGD of the sketch fields runs inside the
           group's backward, in that order, with the optimizer's current learning rate.

`python -m cafe_b200.dlrm_harness --help` trains on seeded synthetic data of a named shape and prints loss, AUC
and samples/s.  torch.autograd.profiler.record_function ranges mark the library calls so that they show up in the
reference's --enable-profiling trace (dlrm_s_pytorch.py:125, 153, 1576-1578).
"""
from __future__ import annotations

import argparse
import time

import numpy as np
import torch
import torch.nn as nn
from torch.autograd.profiler import record_function

from . import sizing, synthetic
from .sk_embedding_bag import SKEmbeddingGroup


def add_cafe_arguments(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    """The CAFE options of the reference's scripts, same names and defaults."""
    parser.add_argument("--sketch-flag", action="store_true", default=False)
    parser.add_argument("--compress-rate", type=float, default=0.001)
    parser.add_argument("--hash-rate", type=float, default=0.5)
    parser.add_argument("--sketch-threshold", type=int, default=1)
    parser.add_argument("--adjust-threshold", type=int, default=1)
    parser.add_argument("--sketch-alpha", type=float, default=1.0)
    parser.add_argument("--notinsert-test", action="store_true", default=False)
    # not a flag of the reference: its dot interaction (dlrm_s_pytorch.py:779-812) as one library kernel per direction
    parser.add_argument("--fused-interaction", action="store_true", default=False)
    return parser


def create_mlp(ln, sigmoid_layer: int, rng: np.random.Generator) -> nn.Sequential:
    """dlrm_s_pytorch.py:213-251: Linear layers with normal(0, sqrt(2/(m+n))) weights and normal(0, sqrt(1/m))
    biases, ReLU after each except a Sigmoid after layer `sigmoid_layer`."""
    layers = []
    for i in range(len(ln) - 1):
        n, m = int(ln[i]), int(ln[i + 1])
        lin = nn.Linear(n, m, bias=True)
        lin.weight.data = torch.from_numpy(rng.normal(0.0, np.sqrt(2 / (m + n)), size=(m, n)).astype(np.float32))
        lin.bias.data = torch.from_numpy(rng.normal(0.0, np.sqrt(1 / m), size=m).astype(np.float32))
        layers.append(lin)
        layers.append(nn.Sigmoid() if i == sigmoid_layer else nn.ReLU())
    return nn.Sequential(*layers)


class CafeEmbeddingLayer(nn.Module):
    """All embedding tables of a model: sketch fields behind one SKEmbeddingGroup, the rest plain tables.

    forward(lS_o, lS_i) takes the reference's per-field offsets / indices (lists or [F, B] tensors, one id per
    bag) and returns [B, F, D] in the original field order."""

    def __init__(self, ln_emb, dim, compress_rate, hash_rate, sketch_threshold=1, adjust_threshold=1, sketch_alpha=1.0,
                 sketch_flag=True, device="cuda", max_batch=4096, lr=0.1, seed=0, notinsert_test=False):
        super().__init__()
        self.ln = [int(n) for n in ln_emb]
        self.dim = int(dim)
        self.device = torch.device(device)
        self.notinsert_test = notinsert_test
        offs = sizing.field_offsets(self.ln)
        self.sketch_fields = [i for i, n in enumerate(self.ln) if sketch_flag and sizing.is_sketch_field(n, compress_rate)]
        self.plain_fields = [i for i in range(len(self.ln)) if i not in self.sketch_fields]
        self.hotn = sizing.hot_rows(sum(self.ln), compress_rate, hash_rate, self.dim) if sketch_flag else 0
        self.group = None
        if self.sketch_fields:
            self.group = SKEmbeddingGroup([self.ln[i] for i in self.sketch_fields], self.dim, compress_rate, hash_rate,
                                          sketch_threshold, adjust_threshold, sketch_alpha, device=self.device,
                                          max_batch=max_batch, lr=lr, f_offsets=[offs[i] for i in self.sketch_fields],
                                          hotn=self.hotn, seed=seed)
        rng = np.random.default_rng(seed + 17)
        self.plain = nn.ModuleList()
        for i in self.plain_fields:
            n = self.ln[i]
            ee = nn.EmbeddingBag(n, self.dim, mode="sum", sparse=True)
            b = np.sqrt(1 / max(n, 5))
            ee.weight.data = torch.from_numpy(rng.uniform(-b, b, size=(n, self.dim)).astype(np.float32))
            self.plain.append(ee)
        self.plain.to(self.device)
        self._arange = None
        self._sk_index = None

    def set_lr(self, lr: float) -> None:
        if self.group is not None:
            self.group.lr = float(lr)

    def forward(self, lS_o, lS_i, test: bool = False) -> torch.Tensor:
        ids = lS_i if isinstance(lS_i, torch.Tensor) else torch.stack(list(lS_i))
        F, B = ids.shape
        cols = [None] * F
        ids = ids.to(self.device, non_blocking=True)         # one copy for all fields
        if self.group is not None:
            with record_function("CAFE sketch fields forward"):
                sk_ids = ids if not self.plain_fields else ids[self._sketch_index()]
                if test:
                    with torch.no_grad():
                        emb = self.group(sk_ids)
                else:
                    emb = self.group(sk_ids)
            if not self.plain_fields:
                return emb                                   # every field goes through the sketch: [B, F, D] as it is
            for j, i in enumerate(self.sketch_fields):
                cols[i] = emb[:, j, :]
        if self._arange is None or self._arange.numel() != B:
            self._arange = torch.arange(B, device=self.device)
        with record_function("plain embedding bags"):
            for j, i in enumerate(self.plain_fields):
                cols[i] = self.plain[j](ids[i], self._arange)
        return torch.stack(cols, dim=1)

    def _sketch_index(self) -> torch.Tensor:
        if self._sk_index is None:
            self._sk_index = torch.tensor(self.sketch_fields, dtype=torch.int64, device=self.device)
        return self._sk_index


class ShardedCafeEmbeddingLayer(nn.Module):
    """The embedding layer of a data-parallel model whose sketch fields are sharded by field over the ranks of a
    process group (ShardedSKEmbedding): every rank feeds the ids of ITS slice of the global batch, [F, B_local], and
    gets back the pooled rows of that slice, [B_local, F, D], in the original field order.  The owners of the fields
    run lookup, sketch insert, migration and SGD for the whole global batch inside backward.

    Fields small enough to be plain tables by the reference's rule (at most 2000 * compress_rate ids,
    dlrm_s_pytorch.py:309) are replicated on every rank, all in one joint table of a few hundred rows: its gradient
    (sparse on each rank, made dense for the exchange) travels with the MLPs' in the step's one all-reduce, and every
    replica applies the same update (for SGD a dense gradient with zero rows for untouched ids equals the
    reference's sparse one).  The hot-row capacity is sized from the sketch fields' ids alone."""

    def __init__(self, ln_emb, dim, compress_rate, hash_rate, sketch_threshold=1, adjust_threshold=1, sketch_alpha=1.0,
                 device="cuda", local_batch=2048, lr=0.1, seed=0, group=None, exchange="peer", **_unused):
        super().__init__()
        import torch.distributed as dist
        from .sharded import ShardedSKEmbedding
        self.ln = [int(n) for n in ln_emb]
        self.dim = int(dim)
        self.device = torch.device(device)
        offs = sizing.field_offsets(self.ln)
        self.sketch_fields = [i for i, n in enumerate(self.ln) if sizing.is_sketch_field(n, compress_rate)]
        self.plain_fields = [i for i in range(len(self.ln)) if i not in self.sketch_fields]
        if not self.sketch_fields:
            raise ValueError("no field is large enough for the sketch at this compress_rate: nothing to shard")
        self.world = dist.get_world_size(group)
        self.local_batch = int(local_batch)
        self.sharded = ShardedSKEmbedding([self.ln[i] for i in self.sketch_fields], self.dim, compress_rate, hash_rate,
                                          sketch_threshold, adjust_threshold, sketch_alpha, device=self.device,
                                          global_batch=self.local_batch * self.world, lr=lr, seed=seed, group=group,
                                          exchange=exchange, f_offsets=[offs[i] for i in self.sketch_fields])
        self.group = self.sharded.group            # this rank's fields (the outer optimizer skips its tables)
        self.hotn = self.group.hotn
        # the plain fields' tables lie one behind the other in ONE parameter (a few hundred rows): one lookup, one
        # sparse gradient and one update per step for all of them.  Same values on every rank, initialised per table
        # as the reference does (dlrm_s_pytorch.py:324-340).
        rng = np.random.default_rng(seed + 17)
        tables, starts, tot = [], [], 0
        for i in self.plain_fields:
            n = self.ln[i]
            b = np.sqrt(1 / max(n, 5))
            tables.append(torch.from_numpy(rng.uniform(-b, b, size=(n, self.dim)).astype(np.float32)))
            starts.append(tot)
            tot += n
        self.plain_weight = None
        if self.plain_fields:
            self.plain_weight = nn.Parameter(torch.cat(tables).to(self.device))
            self.register_buffer("_plain_start", torch.tensor(starts, dtype=torch.int64, device=self.device)[:, None], persistent=False)
            self.register_buffer("_plain_index", torch.tensor(self.plain_fields, dtype=torch.int64, device=self.device), persistent=False)
            order = self.sketch_fields + self.plain_fields           # column c of [sketch | plain] is field order[c]
            place = [order.index(f) for f in range(len(self.ln))]
            self.register_buffer("_place", torch.tensor(place, dtype=torch.int64, device=self.device), persistent=False)
        self._sk_index = torch.tensor(self.sketch_fields, dtype=torch.int64, device=self.device)

    def set_lr(self, lr: float) -> None:
        self.group.lr = float(lr)

    def forward(self, lS_o, lS_i, test: bool = False) -> torch.Tensor:
        ids = lS_i if isinstance(lS_i, torch.Tensor) else torch.stack(list(lS_i))
        ids = ids.to(self.device, non_blocking=True)         # one copy for all fields
        with record_function("CAFE sharded fields forward"):
            sk_ids = ids if not self.plain_fields else ids[self._sk_index]
            if test:
                with torch.no_grad():
                    blocked = self.sharded(sk_ids)
            else:
                blocked = self.sharded(sk_ids)
            emb = self.sharded.plan.unblock(blocked, ids.shape[1], self.dim)
        if not self.plain_fields:
            return emb
        with record_function("plain embedding tables"):
            rows = ids[self._plain_index] + self._plain_start                               # [P, B] rows of the joint table
            pe = nn.functional.embedding(rows, self.plain_weight, sparse=True)               # [P, B, D]
            return torch.cat([emb, pe.transpose(0, 1)], dim=1).index_select(1, self._place)


def dot_interaction(x, emb: torch.Tensor) -> torch.Tensor:
    """dlrm_s_pytorch.py:779-812 (arch_interaction_itself = False): pairwise dot products of the dense vector and
    the embedding vectors, lower triangle, concatenated behind the dense vector."""
    B = emb.shape[0]
    T = emb if x is None else torch.cat([x.unsqueeze(1), emb], dim=1)
    Z = torch.bmm(T, T.transpose(1, 2))
    n = T.shape[1]
    li, lj = torch.tril_indices(n, n, offset=-1, device=emb.device)
    flat = Z[:, li, lj]
    return flat if x is None else torch.cat([x, flat], dim=1)


class _FusedDotInteraction(torch.autograd.Function):
    """dot_interaction as one library kernel per direction (cafe_dot_interaction_forward / _backward): no [B, F+1, F+1]
    intermediate, no index gathers.  x [B, D] and emb [B, F, D] fp32 on the GPU."""

    @staticmethod
    def forward(ctx, x, emb):
        from . import _lib
        lib = _lib.load()
        x, emb = x.contiguous(), emb.contiguous()
        B, F, D = emb.shape
        nv = F + 1
        out = torch.empty(B, D + nv * (nv - 1) // 2, dtype=torch.float32, device=emb.device)
        st = torch.cuda.current_stream(emb.device).cuda_stream
        with torch.cuda.device(emb.device):
            _lib.check(lib.cafe_dot_interaction_forward(x.data_ptr(), emb.data_ptr(), D, F * D, B, F, D, 0, out.data_ptr(),
                                                        out.shape[1], st), "cafe_dot_interaction_forward")
        ctx.save_for_backward(x, emb)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        from . import _lib
        lib = _lib.load()
        x, emb = ctx.saved_tensors
        B, F, D = emb.shape
        g = grad_out.contiguous()
        gx, ge = torch.empty_like(x), torch.empty_like(emb)
        st = torch.cuda.current_stream(emb.device).cuda_stream
        with torch.cuda.device(emb.device):
            _lib.check(lib.cafe_dot_interaction_backward(x.data_ptr(), emb.data_ptr(), D, F * D, B, F, D, 0, g.data_ptr(),
                                                         g.shape[1], gx.data_ptr(), ge.data_ptr(), D, F * D, st),
                       "cafe_dot_interaction_backward")
        return gx, ge


def fused_dot_interaction(x: torch.Tensor, emb: torch.Tensor) -> torch.Tensor:
    """dot_interaction(x, emb) through the library's kernels; same values up to the order of the fp32 additions."""
    if not (x.is_cuda and emb.is_cuda and x.dtype == torch.float32 and emb.dtype == torch.float32):
        raise ValueError("fused_dot_interaction needs fp32 CUDA tensors")
    return _FusedDotInteraction.apply(x, emb)


class DLRMNet(nn.Module):
    """DLRM_Net of dlrm_s_pytorch.py with the CAFE embedding layer: bottom MLP, dot interaction, top MLP.
    `fused_interaction`: the interaction through the library's kernels instead of torch's cat / bmm / index ops."""

    def __init__(self, ln_emb, dim, ln_bot, ln_top_hidden, emb_layer, seed=123, fused_interaction=False):
        super().__init__()
        self.fused_interaction = bool(fused_interaction)
        rng = np.random.default_rng(seed)
        self.emb = emb_layer      # CafeEmbeddingLayer, or anything with the same forward / device / set_lr
        ln_bot = [int(v) for v in ln_bot]
        if ln_bot[-1] != dim:
            raise ValueError("the bottom MLP must end at the embedding dimension")
        self.bot = create_mlp(ln_bot, -1, rng)
        nf = len(ln_emb) + 1
        ln_top = [nf * (nf - 1) // 2 + dim] + [int(v) for v in ln_top_hidden]
        self.top = create_mlp(ln_top, len(ln_top) - 2, rng)
        dev = self.emb.device
        self.bot.to(dev)
        self.top.to(dev)

    def forward(self, dense_x, lS_o, lS_i, test=False):
        with record_function("DLRM forward"):
            x = self.bot(dense_x)
            ly = self.emb(lS_o, lS_i, test)
            if self.fused_interaction and ly.is_cuda:
                return self.top(fused_dot_interaction(x, ly))
            return self.top(dot_interaction(x, ly))


class DCNNet(nn.Module):
    """The deep & cross head of dcn.py:410-422, 712-742 over the CAFE embedding layer: three cross layers
    x_{l+1} = x_0 * (x_l w_l) + b_l, a deep MLP, and a final linear layer over both, then a sigmoid."""

    def __init__(self, ln_emb, dim, num_dense, deep, emb_layer, cross_layers=3, seed=123):
        super().__init__()
        rng = np.random.default_rng(seed)
        self.emb = emb_layer
        self.num_dense = int(num_dense)
        d_in = dim * len(ln_emb) + self.num_dense
        self.deep = create_mlp([d_in] + [int(v) for v in deep], -1, rng)
        g = torch.Generator().manual_seed(seed)
        self.cross_weight = nn.ParameterList([nn.Parameter(torch.randn(d_in, 1, generator=g) * 0.0001) for _ in range(cross_layers)])
        self.cross_bias = nn.ParameterList([nn.Parameter(torch.zeros(d_in)) for _ in range(cross_layers)])
        torch.manual_seed(seed)
        self.last = nn.Linear(d_in + int(deep[-1]), 1)
        dev = self.emb.device
        for m in (self.deep, self.cross_weight, self.cross_bias, self.last):
            m.to(dev)

    def forward(self, dense_x, lS_o, lS_i, test=False):
        with record_function("DLRM forward"):
            ly = self.emb(lS_o, lS_i, test)
            z = ly.reshape(ly.shape[0], -1)
            if self.num_dense:
                z = torch.cat([dense_x, z], dim=1)
            x1 = z
            for w, b in zip(self.cross_weight, self.cross_bias):
                x1 = z * (x1 @ w) + b
            return torch.sigmoid(self.last(torch.cat([self.deep(z), x1], dim=1)))


def dense_and_plain_parameters(model: nn.Module):
    """Everything the outer optimizer updates: MLPs and plain tables.  The sketch fields' tables are updated by the
    group's fused backward (their Parameters never carry a gradient)."""
    skip = set()
    if getattr(model.emb, "group", None) is not None:
        skip = {id(p) for p in model.emb.group.parameters()}
    return [p for p in model.parameters() if id(p) not in skip]


def train_step(model, optimizer, dense_x, lS_o, lS_i, target, loss_fn=None):
    """One step in the reference's order (dlrm_s_pytorch.py:1610-1659).  Returns (loss tensor, predictions)."""
    loss_fn = loss_fn or nn.functional.binary_cross_entropy
    model.emb.set_lr(optimizer.param_groups[0]["lr"])
    z = model(dense_x, lS_o, lS_i, False)
    with record_function("DLRM loss compute"):
        loss = loss_fn(z.squeeze(1), target)
    with record_function("DLRM backward"):
        optimizer.zero_grad()
        # the sketch fields' importance -> insert -> migration -> SGD run inside this backward (insert_grad and the
        # embedding part of optimizer.step of the reference, dlrm_s_pytorch.py:1653-1658)
        loss.backward()
        optimizer.step()
    return loss, z


def allreduce_gradients(params, group=None) -> None:
    """Sums the gradients of `params` over the ranks of `group` in one collective (flattened), in place.  Parameters
    without a gradient are skipped; every rank must hold gradients for the same parameters.  A sparse gradient is
    made dense first (the ranks touch different rows)."""
    import torch.distributed as dist
    for p in params:
        if p.grad is not None and p.grad.is_sparse:      # (small tables looked up with sparse=True)
            p.grad = p.grad.to_dense()
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return
    flat = torch._utils._flatten_dense_tensors(grads)
    dist.all_reduce(flat, group=group)
    for g, f in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
        g.copy_(f)


def train_step_data_parallel(model, optimizer, dense_x, lS_o, lS_i, target, group=None, loss_fn=None):
    """train_step on one rank of a data-parallel job: the rank's loss is its mean over the local batch divided by the
    number of ranks, so that the summed dense gradients and the gradients that reach the embedding owners are those
    of the mean over the GLOBAL batch (one process fed the whole batch would compute the same).  Returns the
    rank's share of the global loss and its predictions."""
    import torch.distributed as dist
    loss_fn = loss_fn or nn.functional.binary_cross_entropy
    world = dist.get_world_size(group)
    model.emb.set_lr(optimizer.param_groups[0]["lr"])
    z = model(dense_x, lS_o, lS_i, False)
    with record_function("DLRM loss compute"):
        loss = loss_fn(z.squeeze(1), target) / world
    with record_function("DLRM backward"):
        optimizer.zero_grad()
        loss.backward()
        allreduce_gradients([p for g in optimizer.param_groups for p in g["params"]], group)
        optimizer.step()
    return loss, z


def auc(y: np.ndarray, p: np.ndarray) -> float:
    order = np.argsort(p, kind="stable")
    y = y[order]
    n1 = float(y.sum())
    n0 = len(y) - n1
    if n1 == 0 or n0 == 0:
        return 0.5
    ranks = np.arange(1, len(y) + 1)
    return float((ranks[y == 1].sum() - n1 * (n1 + 1) / 2) / (n0 * n1))


SHAPES = {
    # name: (cardinalities, dense features, Zipf exponent, label rate, default dim, bottom MLP, top MLP hidden)
    "kaggle": (synthetic.KAGGLE_CARDS, 13, 1.1, 0.25, 16, "13-512-256-64-16", "512-256-1"),
    "terabyte": (synthetic.TERABYTE_CARDS, 13, 1.1, 0.03, 128, "13-512-256-128", "1024-1024-512-256-1"),
    "avazu": (synthetic.AVAZU_CARDS, 0, 1.0, 0.17, 16, "0-16", "1024-1024"),
}


def synthetic_batch(shape: str, batch: int, seed: int, step: int, device):
    """(dense [B,13] or None, offsets, ids [F,B] int64, labels [B]) of the named shape, generated on the host."""
    cards, nd, s, p, *_ = SHAPES[shape]
    ids = torch.from_numpy(synthetic.batch_ids(cards, batch, s, seed, step))
    dense = torch.from_numpy(synthetic.dense_features(batch, seed, step, nd)).to(device) if nd else None
    y = torch.from_numpy(synthetic.labels(batch, p, seed, step)).to(device)
    return dense, None, ids, y


def build_model(args, device="cuda", group_of_ranks=None):
    """The model the arguments name.  `group_of_ranks` = (process group or None for all ranks,): the embedding fields
    sharded over those ranks (ShardedCafeEmbeddingLayer), the dense side replicated; args.mini_batch_size is then the
    batch of ONE rank."""
    cards, nd, _, _, dim_default, bot, top = SHAPES[args.data_set]
    dim = args.arch_sparse_feature_size or dim_default
    emb_kwargs = dict(compress_rate=args.compress_rate, hash_rate=args.hash_rate, sketch_threshold=args.sketch_threshold,
                      adjust_threshold=args.adjust_threshold, sketch_alpha=args.sketch_alpha, sketch_flag=args.sketch_flag,
                      device=device, max_batch=args.mini_batch_size, lr=args.learning_rate, seed=args.numpy_rand_seed,
                      notinsert_test=args.notinsert_test)
    if group_of_ranks is not None:
        emb = ShardedCafeEmbeddingLayer(cards, dim, local_batch=args.mini_batch_size, group=group_of_ranks[0], **{
            k: v for k, v in emb_kwargs.items() if k not in ("sketch_flag", "max_batch", "notinsert_test")})
    else:
        emb = CafeEmbeddingLayer(cards, dim, **emb_kwargs)
    if args.model == "dcn":
        deep = [int(v) for v in (args.arch_mlp_top or top).split("-")]
        return DCNNet(cards, dim, nd, deep, emb, seed=args.numpy_rand_seed)
    ln_bot = [int(v) for v in (args.arch_mlp_bot or bot).split("-")]
    ln_top = [int(v) for v in (args.arch_mlp_top or top).split("-")]
    return DLRMNet(cards, dim, ln_bot, ln_top, emb, seed=args.numpy_rand_seed,
                   fused_interaction=getattr(args, "fused_interaction", False))


def run(args) -> dict:
    """Trains args.nbatches steps on synthetic data of args.data_set; returns losses, AUC and samples/s."""
    dev = torch.device("cuda", torch.cuda.current_device())
    model = build_model(args, dev)
    opt = torch.optim.SGD(dense_and_plain_parameters(model), lr=args.learning_rate)
    B = args.mini_batch_size
    batches = [synthetic_batch(args.data_set, B, 2024, s, dev) for s in range(args.nbatches)]
    losses, preds, ys = [], [], []
    warm = min(args.warmup_batches, max(0, args.nbatches - 1))
    t0 = None
    for s, (dense, lS_o, ids, y) in enumerate(batches):
        if s == warm:
            torch.cuda.synchronize()
            t0 = time.perf_counter()
        loss, z = train_step(model, opt, dense, lS_o, ids, y)
        losses.append(loss.detach())
        preds.append(z.detach().squeeze(1))
        ys.append(y)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    losses = [float(l) for l in losses]
    tail = max(1, len(batches) // 4)
    a = auc(torch.cat(ys[-tail:]).cpu().numpy(), torch.cat(preds[-tail:]).cpu().numpy())
    return {"data_set": args.data_set, "model": args.model, "batch": B, "steps": args.nbatches, "loss_first": losses[0],
            "loss_last": float(np.mean(losses[-tail:])), "auc_last_quarter": a,
            "samples_per_s": (args.nbatches - warm) * B / dt, "ms_per_step": 1e3 * dt / max(1, args.nbatches - warm),
            "sketch_fields": len(model.emb.sketch_fields), "plain_fields": len(model.emb.plain_fields),
            "hot_rows": model.emb.hotn, "losses": losses}


def run_data_parallel(args, group=None) -> dict:
    """run() on every rank of an initialised NCCL process group (one rank per GPU): fields sharded over the ranks,
    dense side replicated with its gradients summed every step, args.mini_batch_size samples per rank and step
    (weak scaling).  Every rank returns the whole job's samples/s, timed on the host between barriers with the
    device drained, the slowest rank's time counting."""
    import torch.distributed as dist
    dev = torch.device("cuda", torch.cuda.current_device())
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    model = build_model(args, dev, group_of_ranks=(group,))
    opt = torch.optim.SGD(dense_and_plain_parameters(model), lr=args.learning_rate)
    B = args.mini_batch_size
    # rank r takes batches r, r + world, ... of the seeded stream: distinct samples on every rank
    batches = [synthetic_batch(args.data_set, B, 2024, s * world + rank, dev) for s in range(args.nbatches)]
    warm = min(args.warmup_batches, max(0, args.nbatches - 1))
    losses = []
    t0 = None
    for s, (dense, lS_o, ids, y) in enumerate(batches):
        if s == warm:
            torch.cuda.synchronize()
            dist.barrier(group)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
        loss, _ = train_step_data_parallel(model, opt, dense, lS_o, ids, y, group)
        losses.append(loss.detach())
    torch.cuda.synchronize()
    dist.barrier(group)
    torch.cuda.synchronize()
    dt = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
    dist.all_reduce(dt, op=dist.ReduceOp.MAX, group=group)
    dt = float(dt.item())
    tot = torch.stack(losses).double()
    dist.all_reduce(tot, group=group)                 # the ranks' shares add up to the global mean
    tot = tot.cpu().numpy()
    tail = max(1, len(batches) // 4)
    # the replicas must have stayed in step: the same dense parameters on every rank
    flat = torch.cat([p.detach().reshape(-1) for p in dense_and_plain_parameters(model)])   # MLPs and plain tables
    lo, hi = flat.clone(), flat.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
    return {"data_set": args.data_set, "model": args.model, "ranks": world, "batch_per_rank": B, "global_batch": B * world,
            "steps": args.nbatches, "loss_first": float(tot[0]), "loss_last": float(tot[-tail:].mean()),
            "samples_per_s": (args.nbatches - warm) * B * world / dt, "ms_per_step": 1e3 * dt / max(1, args.nbatches - warm),
            "sketch_fields": len(model.emb.sketch_fields), "plain_fields": len(model.emb.plain_fields),
            "hot_rows_this_rank": model.emb.hotn, "sketch_fields_this_rank": len(model.emb.sharded.plan.local_fields),
            "replicas_in_step": bool(torch.equal(lo, hi)), "lookups_this_rank": int(model.emb.group.sketch.stats()["lookups"]),
            "losses": [float(v) for v in tot]}


def make_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="DLRM / DCN with CAFE embeddings on synthetic data of a named shape")
    add_cafe_arguments(ap)
    ap.add_argument("--data-set", default="kaggle", choices=sorted(SHAPES))
    ap.add_argument("--model", default="dlrm", choices=["dlrm", "dcn"])
    ap.add_argument("--arch-sparse-feature-size", type=int, default=0)
    ap.add_argument("--arch-mlp-bot", type=str, default="")
    ap.add_argument("--arch-mlp-top", type=str, default="")
    ap.add_argument("--mini-batch-size", type=int, default=128)
    ap.add_argument("--learning-rate", type=float, default=0.1)
    ap.add_argument("--nbatches", type=int, default=200)
    ap.add_argument("--warmup-batches", type=int, default=10)
    ap.add_argument("--numpy-rand-seed", type=int, default=123)
    ap.add_argument("--enable-profiling", action="store_true", default=False)
    return ap


def main(argv=None):
    args = make_parser().parse_args(argv)
    if args.enable_profiling:
        with torch.autograd.profiler.profile(True, use_device="cuda") as prof:
            res = run(args)
        print(prof.key_averages().table(sort_by="self_cpu_time_total", row_limit=25))
    else:
        res = run(args)
    res.pop("losses")
    print(res)


if __name__ == "__main__":
    main()
