"""SKEmbeddingBag and SKEmbeddingGroup: the CAFE compressed embedding on CUDA kernels.

`SKEmbeddingBag` keeps the constructor, `forward`, `insert_grad` and attributes of the reference
module (tricks/sk_embedding_bag.py:26-208) so the reference's model code can construct and call it
unchanged; `SKEmbeddingGroup` is the same path for all sketch fields of a model in one call per
direction (what DLRM_Net.apply_emb / insert_grad loop over, dlrm_s_pytorch.py:653-659, 734-738).

Differences from the reference that a caller can see:
  * ids may be CPU or CUDA tensors (int32/int64); nothing is synchronised with the host in forward;
  * exactly one id per bag, as in the reference (its mask is per bag, :130-150); `offsets` must be
    None or arange(B); other shapes raise;
  * the SGD update of weight_h / weight_hash is applied by the library (the outer optimizer sees no
    gradient for them) unless `fused_update=False`, which materialises the sparse gradients the
    reference's embedding_bag calls would produce so that torch.optim.SGD can apply them;
  * migration copies a hash row into a hot row only when the id is in the main table after its
    field's insert call (the reference indexes weight_h with a global id, out of range, otherwise).
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch
import torch.nn as nn
from torch.nn.parameter import Parameter

from . import _lib, sizing
from .sketch import HotSketch, _stream


def _ptr_array(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _i64_array(vals):
    return (ctypes.c_int64 * len(vals))(*[int(v) for v in vals])


def _i32_array(vals):
    return (ctypes.c_int32 * len(vals))(*[int(v) for v in vals])


def _check_table(t: torch.Tensor, name: str):
    if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
        raise ValueError(f"{name} must be a contiguous fp32 CUDA tensor")


class _FieldSet:
    """Host-side description of a set of fields passed to the C ABI in one call."""

    def __init__(self, sketch: HotSketch, weight_high, weight_hash, f_offset, hash_size, dim):
        self.sketch = sketch
        self.weight_high = weight_high
        self.weight_hash = list(weight_hash)
        self.nf = len(self.weight_hash)
        self.f_offset = _i64_array(f_offset)
        self.hash_size = _i32_array(hash_size)
        self.dim = int(dim)
        self.hotn = int(weight_high.shape[0])

    def ptrs(self):
        _check_table(self.weight_high.data, "weight_high")
        for w in self.weight_hash:
            _check_table(w.data, "weight_hash")
        return _ptr_array([w.data for w in self.weight_hash]), self.weight_high.data.data_ptr()

    def forward(self, ids: torch.Tensor, out: torch.Tensor, field_stride: int, sample_stride: int):
        """ids [nf*B] field-major on the device; returns (gid, row) saved for the backward."""
        lib, sk = self.sketch.lib, self.sketch
        B = ids.numel() // self.nf
        gid = torch.empty(ids.numel(), dtype=torch.int32, device=ids.device)
        row = torch.empty(ids.numel(), dtype=torch.int32, device=ids.device)
        wp, hp = self.ptrs()
        with torch.cuda.device(ids.device):
            _lib.check(lib.cafe_embed_forward(sk.handle, ids.data_ptr(), int(ids.dtype == torch.int64), self.nf, B,
                                              self.f_offset, self.hash_size, wp, hp, self.hotn, self.dim,
                                              out.data_ptr(), field_stride, sample_stride, gid.data_ptr(),
                                              row.data_ptr(), _stream()), "cafe_embed_forward")
        return gid, row

    def resolve(self, ids: torch.Tensor):
        """The sketch probe alone: (gid, row) of ids [nf*B] as forward() would return them, no rows copied."""
        lib, sk = self.sketch.lib, self.sketch
        B = ids.numel() // self.nf
        gid = torch.empty(ids.numel(), dtype=torch.int32, device=ids.device)
        row = torch.empty(ids.numel(), dtype=torch.int32, device=ids.device)
        with torch.cuda.device(ids.device):
            _lib.check(lib.cafe_embed_resolve(sk.handle, ids.data_ptr(), int(ids.dtype == torch.int64), self.nf, B,
                                              self.f_offset, self.hash_size, self.hotn, gid.data_ptr(), row.data_ptr(),
                                              _stream()), "cafe_embed_resolve")
        return gid, row

    def forward_training(self, ids: torch.Tensor, out: torch.Tensor, field_stride: int, sample_stride: int, mode: int):
        """forward() in two kernels with the backward's head start in between: the sketch probe first, then the
        bucket sorts of the insert and the row sort of the scatter are started on the library's side streams, and
        the row gather runs beside them.  Same results as forward()."""
        lib, sk = self.sketch.lib, self.sketch
        B = ids.numel() // self.nf
        gid = torch.empty(ids.numel(), dtype=torch.int32, device=ids.device)
        row = torch.empty(ids.numel(), dtype=torch.int32, device=ids.device)
        wp, hp = self.ptrs()
        with torch.cuda.device(ids.device):
            _lib.check(lib.cafe_embed_resolve(sk.handle, ids.data_ptr(), int(ids.dtype == torch.int64), self.nf, B,
                                              self.f_offset, self.hash_size, self.hotn, gid.data_ptr(), row.data_ptr(),
                                              _stream()), "cafe_embed_resolve")
            _lib.check(lib.cafe_embed_backward_begin(sk.handle, gid.data_ptr(), row.data_ptr(), self.nf, B, self.hash_size,
                                                     wp, hp, self.hotn, self.dim, mode, _stream()), "cafe_embed_backward_begin")
            _lib.check(lib.cafe_embed_gather(sk.handle, row.data_ptr(), self.nf, B, self.hash_size, wp, hp, self.hotn,
                                             self.dim, out.data_ptr(), field_stride, sample_stride, _stream()),
                       "cafe_embed_gather")
        return gid, row

    def importance(self, grad: torch.Tensor, field_stride: int, sample_stride: int, B: int) -> torch.Tensor:
        imp = torch.empty(self.nf * B, dtype=torch.float32, device=grad.device)
        with torch.cuda.device(grad.device):
            _lib.check(self.sketch.lib.cafe_grad_importance(self.sketch.handle, grad.data_ptr(), field_stride,
                                                            sample_stride, self.nf, B, self.dim, imp.data_ptr(),
                                                            _stream()), "cafe_grad_importance")
        return imp

    def migrate(self, ids, mask, post_row, B):
        wp, hp = self.ptrs()
        with torch.cuda.device(ids.device):
            _lib.check(self.sketch.lib.cafe_migrate(self.sketch.handle, ids.data_ptr(), int(ids.dtype == torch.int64),
                                                    mask.data_ptr(), post_row.data_ptr(), self.nf, B, self.f_offset,
                                                    self.hash_size, wp, hp, self.hotn, self.dim, None, _stream()),
                       "cafe_migrate")

    def scatter_sgd(self, grad, field_stride, sample_stride, row, B, lr):
        wp, hp = self.ptrs()
        with torch.cuda.device(grad.device):
            _lib.check(self.sketch.lib.cafe_scatter_sgd(self.sketch.handle, grad.data_ptr(), field_stride, sample_stride,
                                                        row.data_ptr(), self.nf, B, self.hash_size, wp, hp, self.hotn,
                                                        self.dim, float(lr), _stream()), "cafe_scatter_sgd")

    def backward_begin(self, gid, row, B, mode):
        """Starts the part of the backward that needs only the forward's outputs (the bucket sorts of the
        sketch insert and the row sort of the scatter) on the library's side streams."""
        wp, hp = self.ptrs()
        with torch.cuda.device(gid.device):
            _lib.check(self.sketch.lib.cafe_embed_backward_begin(
                self.sketch.handle, gid.data_ptr(), row.data_ptr(), self.nf, B, self.hash_size, wp, hp, self.hotn,
                self.dim, mode, _stream()), "cafe_embed_backward_begin")

    def backward_gated(self, grad, field_stride, sample_stride, ids, gid, row, B, lr, mode, gate_field, gate_event):
        """backward() whose gradient rows of the fields from gate_field on are complete only once gate_event
        (a torch.cuda.Event recorded on another stream) has fired."""
        wp, hp = self.ptrs()
        with torch.cuda.device(grad.device):
            return _lib.check(self.sketch.lib.cafe_embed_backward_gated(
                self.sketch.handle, grad.data_ptr(), field_stride, sample_stride, ids.data_ptr(),
                int(ids.dtype == torch.int64), gid.data_ptr(), row.data_ptr(), self.nf, B, self.f_offset, self.hash_size,
                wp, hp, self.hotn, self.dim, float(lr), mode, int(gate_field), ctypes.c_void_p(gate_event.cuda_event),
                _stream()), "cafe_embed_backward_gated")

    def backward_norms(self, grad, field_stride, sample_stride, norms, ids, gid, row, B, lr, mode, gate_event=None):
        """backward() from per-lookup gradient norms that are already there ([F, B] fp32) while the gradient rows may
        still be arriving: the stream waits for gate_event (a torch.cuda.Event, or None) only before the SGD scatter."""
        wp, hp = self.ptrs()
        with torch.cuda.device(grad.device):
            return _lib.check(self.sketch.lib.cafe_embed_backward_norms(
                self.sketch.handle, grad.data_ptr(), field_stride, sample_stride, norms.data_ptr(), ids.data_ptr(),
                int(ids.dtype == torch.int64), gid.data_ptr(), row.data_ptr(), self.nf, B, self.f_offset, self.hash_size,
                wp, hp, self.hotn, self.dim, float(lr), mode,
                ctypes.c_void_p(gate_event.cuda_event) if gate_event is not None else None, _stream()),
                "cafe_embed_backward_norms")

    def backward(self, grad, field_stride, sample_stride, ids, gid, row, B, lr, mode, mask_out=None):
        wp, hp = self.ptrs()
        with torch.cuda.device(grad.device):
            return _lib.check(self.sketch.lib.cafe_embed_backward(
                self.sketch.handle, grad.data_ptr(), field_stride, sample_stride, ids.data_ptr(),
                int(ids.dtype == torch.int64), gid.data_ptr(), row.data_ptr(), self.nf, B, self.f_offset, self.hash_size,
                wp, hp, self.hotn, self.dim, float(lr), mode, mask_out.data_ptr() if mask_out is not None else None,
                None, _stream()), "cafe_embed_backward")


def _device_ids(input: torch.Tensor, device) -> torch.Tensor:
    if input.dtype not in (torch.int32, torch.int64):
        raise TypeError("ids must be int32 or int64")
    return input.to(device, non_blocking=True).contiguous()


def _check_offsets(offsets, B):
    if offsets is None:
        return
    if offsets.numel() != B or (B > 0 and (int(offsets[0]) != 0 or int(offsets[-1]) != B - 1)):
        raise ValueError("SKEmbeddingBag supports exactly one id per bag (offsets = arange(B)), like the reference")


class _BagFunction(torch.autograd.Function):
    """out = selected rows; backward leaves the gradient rows with the module (fused update) or
    returns the reference's sparse gradients (fused_update=False)."""

    @staticmethod
    def forward(ctx, weight_h, weight_hash, module, ids):
        B = ids.numel()
        out = torch.empty(B, module.embedding_dim, dtype=torch.float32, device=ids.device)
        gid, row = module._fields.forward(ids, out, 0, module.embedding_dim)
        ctx.module = module
        ctx.save_for_backward(row)
        module._saved = dict(ids=ids, gid=gid, row=row, grad=None)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        m = ctx.module
        (row,) = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        if m._saved is not None and m._saved["row"] is row:
            m._saved["grad"] = grad_out
        if m.fused_update:
            return None, None, None, None
        # the reference's two embedding_bag(sparse=True) backwards under torch.where (:134-150)
        hot = row < 0
        zeros = torch.zeros_like(grad_out)
        idx_h = torch.where(hot, -row, torch.zeros_like(row)).long()
        idx_c = torch.where(hot, torch.zeros_like(row), row).long()
        g_h = torch.sparse_coo_tensor(idx_h[None], torch.where(hot[:, None], grad_out, zeros), m.weight_h.shape)
        g_c = torch.sparse_coo_tensor(idx_c[None], torch.where(hot[:, None], zeros, grad_out), m.weight_hash.shape)
        return g_h, g_c, None, None


class SKEmbeddingBag(nn.Module):
    """Drop-in for tricks/sk_embedding_bag.py:26 (same positional constructor arguments).

    `lib` is the loaded libcafe_b200 (ctypes.CDLL) on which the model has called `init(hotn, threshold,
    adjust, alpha)` as DLRM_Net does (dlrm_s_pytorch.py:444-449), or a `cafe_b200.HotSketch`."""

    def __init__(self, field_num, hotn, lib, weight_high, device, num_categories, embedding_dim, f_offset, hash_size,
                 max_norm=None, norm_type=2.0, scale_grad_by_freq=False, sparse=False, fused_update=True, lr=None):
        super().__init__()
        self.field_num = field_num
        self.lib = lib
        self.offset = int(f_offset)
        self.hash_size = int(hash_size)
        self.hot_nums = int(hotn)
        self.num_categories = int(num_categories)
        self.weight_h = weight_high
        self.embedding_dim = int(embedding_dim)
        self.max_norm, self.norm_type, self.scale_grad_by_freq, self.sparse = max_norm, norm_type, scale_grad_by_freq, sparse
        self.device = torch.device(device)
        self.fused_update = fused_update
        self.lr = lr
        self.query_dic = None
        if not weight_high.is_cuda:
            raise ValueError("weight_high must live on the CUDA device (there is no CPU path)")
        if isinstance(lib, HotSketch):
            self.sketch = lib
        else:
            h = lib.cafe_global_handle()
            if not h:
                raise RuntimeError("lib.init(hotn, threshold, adjust_thres, alpha) must be called before building modules")
            self.sketch = HotSketch(hotn, device=weight_high.device, handle=h)
        if self.sketch.hotn != self.hot_nums:
            raise ValueError("the sketch was initialised for a different number of hot rows")
        self.weight_hash = Parameter(torch.empty(self.hash_size, self.embedding_dim, device=weight_high.device))
        self.reset_parameters()
        self._fields = _FieldSet(self.sketch, self.weight_h, [self.weight_hash], [self.offset], [self.hash_size],
                                 self.embedding_dim)
        self._saved = None

    def reset_parameters(self):
        b = float(np.sqrt(1 / self.num_categories))
        nn.init.uniform_(self.weight_hash, -b, b)

    def query(self, input):
        """(dic_mask, dic) as in the reference's query(): hot flag and |query result|, on the device."""
        ids = _device_ids(input, self.weight_h.device)
        q = self.sketch.query((ids + self.offset).to(torch.int32))
        return q < 0, q.abs()

    def forward(self, input, offsets=None, per_sample_weights=None, test=False):
        ids = _device_ids(input, self.weight_h.device)
        _check_offsets(offsets, ids.numel())
        out = _BagFunction.apply(self.weight_h, self.weight_hash, self, ids)
        self.query_dic = self._saved["row"] < 0
        return out

    def insert_grad(self, input):
        """Importance -> sketch insert -> migration for this field (tricks/sk_embedding_bag.py:173-208).
        Must follow the backward pass of the forward it belongs to."""
        s = self._saved
        if s is None or s["grad"] is None:
            raise RuntimeError("insert_grad() needs the gradient of the last forward(); call it after backward()")
        B, D = s["ids"].numel(), self.embedding_dim
        imp = self._fields.importance(s["grad"], 0, D, B)
        mask, post = self.sketch.insert(s["gid"], imp, [0, B])
        self._fields.migrate(s["ids"], mask, post, B)
        self.last_mask = mask
        return mask

    def apply_update(self, lr=None):
        """row -= lr * sum of its gradient rows, with the rows chosen at forward time (fused mode)."""
        s = self._saved
        if s is None or s["grad"] is None:
            return
        lr = self.lr if lr is None else lr
        if lr is None:
            raise ValueError("learning rate not set")
        B, D = s["ids"].numel(), self.embedding_dim
        with torch.no_grad():
            self._fields.scatter_sgd(s["grad"], 0, D, s["row"], B, lr)
        self._saved = None

    def extra_repr(self):
        return f"{self.num_categories}, {self.embedding_dim}, hash_size={self.hash_size}, hot_rows={self.hot_nums}"


def attach_optimizer(optimizer: torch.optim.Optimizer, modules) -> None:
    """After every optimizer.step(), apply the fused SGD update of the given SKEmbeddingBag modules with
    the learning rate of the optimizer's first parameter group (dlrm_s_pytorch.py:1658 keeps one group)."""
    mods = [m for m in modules if isinstance(m, SKEmbeddingBag) and m.fused_update]

    def _hook(opt, args, kwargs):
        lr = opt.param_groups[0]["lr"]
        for m in mods:
            m.apply_update(lr)

    optimizer.register_step_post_hook(_hook)


class _GroupFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, anchor, group, ids):
        F, B = ids.shape
        out = torch.empty(B, F, group.embedding_dim, dtype=torch.float32, device=ids.device)
        flat = ids.reshape(-1)
        if group.training and ctx.needs_input_grad[0] and flat.numel() > 0:
            # the backward's sorts start right behind the sketch probe and overlap the gather and whatever runs
            # before the backward
            gid, row = group._fields.forward_training(flat, out, group.embedding_dim, F * group.embedding_dim, group.insert_mode)
        else:
            gid, row = group._fields.forward(flat, out, group.embedding_dim, F * group.embedding_dim)
        ctx.group = group
        ctx.saved = (flat, gid, row, B)
        group.last_rows = row.view(F, B)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        g = ctx.group
        flat, gid, row, B = ctx.saved
        F, D = g.num_fields, g.embedding_dim
        grad_out = grad_out.contiguous()
        with torch.no_grad():
            g.last_status = g._fields.backward(grad_out, D, F * D, flat, gid, row, B, g.lr, g.insert_mode)
        return None, None, None


class SKEmbeddingGroup(nn.Module):
    """All sketch fields of a model behind one forward and one backward call.

    Owns what DLRM_Net owns for CAFE (dlrm_s_pytorch.py:438-449, 309-322): the shared hot table, one
    hash table per field and the sketch.  forward(ids[F,B]) -> [B,F,D]; its backward runs, in the
    reference's order, importance -> insert (one call per field, ascending) -> migration -> SGD with
    learning rate `self.lr`, in place.  Parameters therefore never carry a .grad."""

    def __init__(self, num_categories, embedding_dim, compress_rate, hash_rate, sketch_threshold=1, adjust_threshold=1,
                 sketch_alpha=1.0000005, device="cuda", max_batch=65536, lr=0.1, f_offsets=None, hotn=None,
                 total_categories=None, insert_mode=_lib.INSERT_PARALLEL, seed=None):
        super().__init__()
        self.num_categories = [int(n) for n in num_categories]
        self.num_fields = len(self.num_categories)
        if not 1 <= self.num_fields <= _lib.MAX_FIELDS:
            raise ValueError(f"1..{_lib.MAX_FIELDS} fields per group")
        self.embedding_dim = int(embedding_dim)
        self.lr = float(lr)
        self.insert_mode = insert_mode
        dev = torch.device(device)
        if dev.type != "cuda":
            raise ValueError("SKEmbeddingGroup needs a CUDA device; there is no CPU path")
        if dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        totn = int(total_categories) if total_categories is not None else sum(self.num_categories)
        self.hotn = int(hotn) if hotn is not None else sizing.hot_rows(totn, compress_rate, hash_rate, self.embedding_dim)
        self.hash_sizes = [sizing.hash_rows(n, compress_rate, hash_rate) for n in self.num_categories]
        self.f_offsets = list(f_offsets) if f_offsets is not None else sizing.field_offsets(self.num_categories)
        gen = torch.Generator(device="cpu")
        if seed is not None:
            gen.manual_seed(seed)
        # the reference leaves weight_high uninitialised (dlrm_s_pytorch.py:439-442); use the artifact
        # tree's choice, uniform(+-sqrt(1/max n)) (ArtifactEvaluation/embeddings/init_embed.py:119-120)
        bh = float(np.sqrt(1 / max(self.num_categories)))
        self.weight_high = Parameter(((torch.rand(self.hotn, self.embedding_dim, generator=gen) * 2 - 1) * bh).to(dev))
        self.weight_hash = nn.ParameterList()
        for n, hs in zip(self.num_categories, self.hash_sizes):
            b = float(np.sqrt(1 / n))
            self.weight_hash.append(Parameter(((torch.rand(hs, self.embedding_dim, generator=gen) * 2 - 1) * b).to(dev)))
        self.sketch = HotSketch(self.hotn, sketch_threshold, adjust_threshold, sketch_alpha,
                                max_lookups=max(1, self.num_fields * int(max_batch)), device=dev)
        self._fields = _FieldSet(self.sketch, self.weight_high, list(self.weight_hash), self.f_offsets, self.hash_sizes,
                                 self.embedding_dim)
        self._anchor = Parameter(torch.zeros(1, device=dev))   # gives the autograd node an input that requires grad
        self.last_status = 0
        self.last_rows = None

    # ---- checkpointing: the sketch travels with the module's state_dict ----------------------------------
    # (the reference cannot resume a CAFE run: its sketch state is never saved and the lib.update() it calls
    # on load does not exist, dlrm_s_pytorch.py:1488-1511)
    def get_extra_state(self):
        st = self.sketch.state()
        return {k: (torch.from_numpy(v.astype(np.int64) if v.dtype == np.uint32 else v) if isinstance(v, np.ndarray) else v)
                for k, v in st.items()}

    def set_extra_state(self, state):
        st = {}
        for k, v in state.items():
            if isinstance(v, torch.Tensor):
                a = v.cpu().numpy()
                st[k] = a.astype(np.uint32) if k in ("main_val", "lru_val", "queue") else a
            else:
                st[k] = v
        self.sketch.load_state(st)

    def row_codes(self, ids: torch.Tensor) -> torch.Tensor:
        """int32 [num_fields, batch]: the table row every lookup of ids [num_fields, batch] reads right now: -r for row r
        of the shared hot table, otherwise the row of the field's own hash table (sk_embedding_bag.py:141-153)."""
        ids = _device_ids(ids, self.weight_high.device)
        with torch.no_grad():
            return self._fields.resolve(ids.reshape(-1))[1].view(self.num_fields, -1)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        if ids.dim() != 2 or ids.shape[0] != self.num_fields:
            raise ValueError("ids must be [num_fields, batch]")
        ids = _device_ids(ids, self.weight_high.device)
        if ids.numel() > self.sketch.capacity:
            raise ValueError("batch larger than max_batch given at construction")
        return _GroupFunction.apply(self._anchor, self, ids)
