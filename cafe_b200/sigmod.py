"""The one-stage HotSketch policy of the reference's artifact tree on the same CUDA path.

`SigmodSketch` stands in for the ctypes use of ArtifactEvaluation/embeddings/sketch.cpp (init / batch_query /
batch_insert / batch_insert_val / update, :124-150, 222-230; one sketch per `idx`, here one object per sketch);
`SigmodSKEmbeddingBag` keeps the constructor, forward and insert_grad of that tree's module
(ArtifactEvaluation/embeddings/sk_embedding_bag.py:11-180), with the data path of cafe_b200.SKEmbeddingBag: rows
are gathered by cafe_embed_gather from the row codes of cafe_sigmod_resolve, importance / migration / SGD are the
same kernels as for the CAFE+ sketch.  Ids may be CPU or CUDA tensors; there is no CPU path.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch
import torch.nn as nn
from torch.nn.parameter import Parameter

from . import _lib
from .sketch import _stream


class SigmodSketch:
    """init(n, Threshold, dr, idx) of ArtifactEvaluation/embeddings/sketch.cpp:228-230 as an object."""

    def __init__(self, lim: int, threshold: int, decay_rate: float = 0.99, max_lookups: int = 1 << 16, device=None):
        if not torch.cuda.is_available():
            raise RuntimeError("cafe_b200.SigmodSketch needs a CUDA device; there is no CPU fallback")
        self.lib = _lib.load()
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        h = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.cafe_sigmod_create(ctypes.byref(h), int(lim), int(threshold), float(decay_rate),
                                                   int(max_lookups)), "cafe_sigmod_create")
        self.handle, self.lim, self.threshold, self.capacity = h.value, int(lim), int(threshold), int(max_lookups)

    def close(self):
        if getattr(self, "handle", None):
            self.lib.cafe_sigmod_destroy(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ids(self, gid: torch.Tensor) -> torch.Tensor:
        gid = gid.to(self.device)
        return (gid if gid.dtype == torch.int32 else gid.to(torch.int32)).contiguous()

    def query(self, gid: torch.Tensor) -> torch.Tensor:
        gid = self._ids(gid)
        out = torch.empty_like(gid)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.cafe_sigmod_query(self.handle, gid.data_ptr(), gid.numel(), out.data_ptr(), _stream()),
                       "cafe_sigmod_query")
        return out

    def insert(self, gid: torch.Tensor, imp: torch.Tensor | None) -> torch.Tensor:
        """batch_insert_val (batch_insert when imp is None): the per-lookup result (1 = handed a hot row)."""
        gid = self._ids(gid)
        mask = torch.empty(gid.numel(), dtype=torch.int32, device=self.device)
        ip = None
        if imp is not None:
            imp = imp.to(device=self.device, dtype=torch.float32).contiguous()
            if imp.numel() != gid.numel():
                raise ValueError("one importance per id")
            ip = imp.data_ptr()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.cafe_sigmod_insert(self.handle, gid.data_ptr(), ip, gid.numel(), mask.data_ptr(), _stream()),
                       "cafe_sigmod_insert")
        return mask

    def update(self) -> None:
        with torch.cuda.device(self.device):
            _lib.check(self.lib.cafe_sigmod_update(self.handle, _stream()), "cafe_sigmod_update")

    # numpy conveniences with the oracle's method names (parity tests)
    def _np(self, ids):
        return torch.from_numpy(np.ascontiguousarray(np.asarray(ids).astype(np.uint32)).view(np.int32)).to(self.device)

    def batch_query(self, ids) -> np.ndarray:
        return self.query(self._np(ids)).cpu().numpy()

    def batch_insert_val(self, ids, v=None) -> np.ndarray:
        vi = None if v is None else torch.from_numpy(np.ascontiguousarray(v, np.float32)).to(self.device)
        return self.insert(self._np(ids), vi).cpu().numpy()

    def batch_insert(self, ids) -> np.ndarray:
        return self.batch_insert_val(ids, None)

    def state(self) -> dict:
        n = self.lim
        val, cnt, dic = np.zeros(n * 4, np.uint32), np.zeros(n * 4, np.float32), np.zeros(n * 4, np.int32)
        q, s, tot = np.zeros(n, np.uint32), np.zeros(3, np.int64), ctypes.c_double()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.cafe_sigmod_dump(self.handle, val.ctypes.data_as(_lib._u32p), cnt.ctypes.data_as(_lib._f32p),
                                                 dic.ctypes.data_as(_lib._i32p), q.ctypes.data_as(_lib._u32p),
                                                 s.ctypes.data_as(_lib._i64p), ctypes.byref(tot), _stream()), "cafe_sigmod_dump")
        return dict(num=int(s[0]), tot=tot.value, decays=int(s[2]), val=val, cnt=cnt, dic=dic, queue=q[:int(s[1])].copy())

    def load_state(self, st: dict) -> None:
        val, cnt, dic = (np.ascontiguousarray(st["val"], np.uint32), np.ascontiguousarray(st["cnt"], np.float32),
                         np.ascontiguousarray(st["dic"], np.int32))
        if val.size != self.lim * 4:
            raise ValueError("state was saved from a sketch of another size")
        with torch.cuda.device(self.device):
            _lib.check(self.lib.cafe_sigmod_load(self.handle, val.ctypes.data_as(_lib._u32p), cnt.ctypes.data_as(_lib._f32p),
                                                 dic.ctypes.data_as(_lib._i32p), int(st["num"]), float(st["tot"]), _stream()),
                       "cafe_sigmod_load")


class _Workspace:
    """Handle without a sketch that carries the scratch of the importance / migration / scatter entry points."""

    def __init__(self, hotn: int, max_lookups: int, device):
        self.lib = _lib.load()
        h = ctypes.c_void_p()
        with torch.cuda.device(device):
            _lib.check(self.lib.cafe_workspace_create(ctypes.byref(h), int(hotn), int(max_lookups)), "cafe_workspace_create")
        self.handle = h.value

    def __del__(self):
        try:
            if self.handle:
                self.lib.cafe_sketch_destroy(self.handle)
        except Exception:
            pass


class _SigmodBagFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, weight_h, weight_hash, module, ids):
        B = ids.numel()
        lib = module.sketch.lib
        out = torch.empty(B, module.embedding_dim, dtype=torch.float32, device=ids.device)
        gid = torch.empty(B, dtype=torch.int32, device=ids.device)
        row = torch.empty(B, dtype=torch.int32, device=ids.device)
        hs = (ctypes.c_int32 * 1)(module.hash_size)
        wp = (ctypes.c_void_p * 1)(module.weight_hash.data.data_ptr())
        with torch.cuda.device(ids.device):
            _lib.check(lib.cafe_sigmod_resolve(module.sketch.handle, ids.data_ptr(), int(ids.dtype == torch.int64), module.offset,
                                               module.hash_size, B, gid.data_ptr(), row.data_ptr(), _stream()),
                       "cafe_sigmod_resolve")
            _lib.check(lib.cafe_embed_gather(module._ws.handle, row.data_ptr(), 1, B, hs, wp, module.weight_h.data.data_ptr(),
                                             module.hot_nums, module.embedding_dim, out.data_ptr(), 0, module.embedding_dim,
                                             _stream()), "cafe_embed_gather")
        ctx.module = module
        module._saved = dict(ids=ids, gid=gid, row=row, grad=None)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        m = ctx.module
        if m._saved is not None:
            m._saved["grad"] = grad_out.contiguous()
        return None, None, None, None


class SigmodSKEmbeddingBag(nn.Module):
    """Drop-in for ArtifactEvaluation/embeddings/sk_embedding_bag.py:11 (same positional constructor arguments, with
    `lib` a SigmodSketch: the per-field one when cafe_hot_separate_field is set, else the one all fields share).

    forward(input, offsets) as in the reference (one id per bag); insert_grad(input, use_freq) runs importance ->
    sketch insert -> migration; apply_update(lr) applies the SGD step of the rows chosen at forward time (the
    reference leaves that to its optimizer)."""

    def __init__(self, field_idx, hotn, lib, weight_high, device, num_categories, embedding_dim, f_offset, hash_size,
                 cafe_hot_separate_field=False, max_batch=65536):
        super().__init__()
        if not isinstance(lib, SigmodSketch):
            raise TypeError("lib must be a cafe_b200.sigmod.SigmodSketch")
        if lib.lim != int(hotn):
            raise ValueError("the sketch was created for a different number of hot rows")
        self.field_idx, self.ss_idx = field_idx, (field_idx if cafe_hot_separate_field else 0)
        self.cafe_hot_separate_field = cafe_hot_separate_field
        self.sketch, self.lib = lib, lib
        self.offset, self.hash_size, self.hot_nums = int(f_offset), int(hash_size), int(hotn)
        self.num_categories, self.embedding_dim = int(num_categories), int(embedding_dim)
        self.weight_h = weight_high
        self.device = torch.device(device)
        if not weight_high.is_cuda:
            raise ValueError("weight_high must live on the CUDA device (there is no CPU path)")
        self.weight_hash = Parameter(torch.empty(self.hash_size, self.embedding_dim, device=weight_high.device))
        b = float(np.sqrt(1 / self.num_categories))
        nn.init.uniform_(self.weight_hash, -b, b)
        self._ws = _Workspace(self.hot_nums, max_batch, weight_high.device)
        self._saved = None
        self.query_dic = None

    def forward(self, input, offsets=None):
        ids = input.to(self.weight_h.device, non_blocking=True).contiguous()
        if ids.dtype not in (torch.int32, torch.int64):
            raise TypeError("ids must be int32 or int64")
        if offsets is not None and offsets.numel() != ids.numel():
            raise ValueError("exactly one id per bag (offsets = arange(B)), like the reference")
        out = _SigmodBagFunction.apply(self.weight_h, self.weight_hash, self, ids)
        self.query_dic = self._saved["row"] < 0
        return out

    def insert_grad(self, input, use_freq=False):
        s = self._saved
        if s is None or (s["grad"] is None and not use_freq):
            raise RuntimeError("insert_grad() needs the gradient of the last forward(); call it after backward()")
        B, D, lib = s["ids"].numel(), self.embedding_dim, self.sketch.lib
        dev = self.weight_h.device
        with torch.cuda.device(dev):
            if use_freq:
                imp = None     # the reference passes ones (:148-149): batch_insert_val with unit counts == batch_insert
            else:
                imp = torch.empty(B, dtype=torch.float32, device=dev)
                _lib.check(lib.cafe_grad_importance(self._ws.handle, s["grad"].data_ptr(), 0, D, 1, B, D, imp.data_ptr(),
                                                    _stream()), "cafe_grad_importance")
            mask = self.sketch.insert(s["gid"], imp)
            post = torch.empty(B, dtype=torch.int32, device=dev)
            _lib.check(lib.cafe_sigmod_post_rows(self.sketch.handle, s["gid"].data_ptr(), mask.data_ptr(), B, post.data_ptr(),
                                                 _stream()), "cafe_sigmod_post_rows")
            hs = (ctypes.c_int32 * 1)(self.hash_size)
            off = (ctypes.c_int64 * 1)(self.offset)
            wp = (ctypes.c_void_p * 1)(self.weight_hash.data.data_ptr())
            _lib.check(lib.cafe_migrate(self._ws.handle, s["ids"].data_ptr(), int(s["ids"].dtype == torch.int64), mask.data_ptr(),
                                        post.data_ptr(), 1, B, off, hs, wp, self.weight_h.data.data_ptr(), self.hot_nums, D, None,
                                        _stream()), "cafe_migrate")
        self.last_mask = mask
        return mask

    def apply_update(self, lr: float):
        s = self._saved
        if s is None or s["grad"] is None:
            return
        B, D, lib = s["ids"].numel(), self.embedding_dim, self.sketch.lib
        hs = (ctypes.c_int32 * 1)(self.hash_size)
        wp = (ctypes.c_void_p * 1)(self.weight_hash.data.data_ptr())
        with torch.no_grad(), torch.cuda.device(self.weight_h.device):
            _lib.check(lib.cafe_scatter_sgd(self._ws.handle, s["grad"].data_ptr(), 0, D, s["row"].data_ptr(), 1, B, hs, wp,
                                            self.weight_h.data.data_ptr(), self.hot_nums, D, float(lr), _stream()),
                       "cafe_scatter_sgd")
        self._saved = None
