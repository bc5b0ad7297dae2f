"""HotSketch: the device-resident CAFE+ sketch behind a small Python class.

Stands in for the ctypes use of the reference's sklib.so (tricks/sk_embedding_bag.py:61-73,
dlrm_s_pytorch.py:444-449), but with device tensors in and out and one handle per sketch so that a
process can hold several (one per shard).
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _lib

STAT_NAMES = ["calls", "lookups", "rounds", "jobs", "truncated_jobs", "resets", "resets_refused", "flips",
              "seq_fallbacks", "main_hits", "lru_visits", "events", "max_rounds"]
_STATE_ARRAYS = ["main_val", "main_cnt", "main_dic", "main_flip", "lru_val", "lru_cnt", "lru_dic", "lru_t",
                 "lru_flip", "queue"]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _np_ptr(a: np.ndarray, typ):
    return a.ctypes.data_as(typ)


class HotSketch:
    """init(n, Threshold, adjust_thres, alp) of tricks/sketch.cpp:309-313, as an object."""

    def __init__(self, hotn: int, threshold: float = 1, adjust_thres: int = 1, alpha: float = 1.0000005,
                 max_lookups: int = 1 << 20, device=None, handle: int | None = None):
        if not torch.cuda.is_available():
            raise RuntimeError("cafe_b200.HotSketch needs a CUDA device; there is no CPU fallback")
        self.lib = _lib.load()
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self._owned = handle is None
        if handle is None:
            h = ctypes.c_void_p()
            with torch.cuda.device(self.device):
                _lib.check(self.lib.cafe_sketch_create(ctypes.byref(h), int(hotn), float(threshold), int(adjust_thres),
                                                       float(alpha), int(max_lookups)), "cafe_sketch_create")
            self.handle = h.value
        else:
            self.handle = handle
        n1, n2, lim, cap = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        self.lib.cafe_sketch_sizes(self.handle, ctypes.byref(n1), ctypes.byref(n2), ctypes.byref(lim), ctypes.byref(cap))
        self.n1, self.n2, self.hotn, self.capacity = n1.value, n2.value, lim.value, cap.value
        self.last_status = 0

    def close(self):
        if getattr(self, "handle", None) and self._owned:
            self.lib.cafe_sketch_destroy(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- reference calls -------------------------------------------------------------------------
    def _ids(self, gid: torch.Tensor) -> torch.Tensor:
        if gid.device != self.device:
            gid = gid.to(self.device)
        if gid.dtype != torch.int32:
            gid = gid.to(torch.int32)   # same 32 bits as the reference's astype(np.int32)
        return gid.contiguous()

    def query(self, gid: torch.Tensor) -> torch.Tensor:
        """batch_query: -hot_row where hot, else the id (int32)."""
        gid = self._ids(gid)
        out = torch.empty_like(gid)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.cafe_sketch_query(self.handle, gid.data_ptr(), gid.numel(), out.data_ptr(), _stream()),
                       "cafe_sketch_query")
        return out

    def insert(self, gid: torch.Tensor, imp: torch.Tensor | None, seg_off=None, mode: int = _lib.INSERT_PARALLEL,
               want_post_row: bool = True):
        """One batch_insert_val (batch_insert if imp is None) per segment.  Returns (mask, post_row)."""
        gid = self._ids(gid)
        n = gid.numel()
        if seg_off is None:
            seg_off = [0, n]
        seg = (ctypes.c_int * len(seg_off))(*[int(x) for x in seg_off])
        if int(seg_off[-1]) != n:
            raise ValueError("segment offsets must end at the number of ids")
        mask = torch.empty(n, dtype=torch.int32, device=self.device)
        post = torch.empty(n, dtype=torch.int32, device=self.device) if want_post_row else None
        impp = None
        if imp is not None:
            imp = imp.to(device=self.device, dtype=torch.float32).contiguous()
            if imp.numel() != n:
                raise ValueError("one importance per id")
            impp = imp.data_ptr()
        with torch.cuda.device(self.device):
            self.last_status = _lib.check(
                self.lib.cafe_sketch_insert(self.handle, gid.data_ptr(), impp, seg, len(seg_off) - 1, mask.data_ptr(),
                                            post.data_ptr() if post is not None else None, mode, _stream()),
                "cafe_sketch_insert")
        return mask, post

    def refit(self) -> int:
        with torch.cuda.device(self.device):
            return _lib.check(self.lib.cafe_sketch_refit(self.handle, _stream()), "cafe_sketch_refit")

    def tune(self, window: int = 0, round_cap: int = 0):
        self.lib.cafe_sketch_tuning(self.handle, window, round_cap)

    # ---- numpy conveniences with the oracle's method names (used by parity tests) -----------------
    def batch_query(self, ids) -> np.ndarray:
        t = torch.from_numpy(np.ascontiguousarray(np.asarray(ids).astype(np.uint32)).view(np.int32)).to(self.device)
        return self.query(t).cpu().numpy()

    def batch_insert_val(self, ids, v=None, mode: int = _lib.INSERT_PARALLEL) -> np.ndarray:
        t = torch.from_numpy(np.ascontiguousarray(np.asarray(ids).astype(np.uint32)).view(np.int32)).to(self.device)
        vi = None if v is None else torch.from_numpy(np.ascontiguousarray(v, np.float32)).to(self.device)
        mask, _ = self.insert(t, vi, None, mode, want_post_row=False)
        return mask.cpu().numpy()

    # ---- state ------------------------------------------------------------------------------------
    def scalars(self) -> dict:
        s = np.zeros(8, np.int64)
        dec = ctypes.c_double()
        self.lib.cafe_sketch_scalars(self.handle, _np_ptr(s, _lib._i64p), ctypes.byref(dec))
        return dict(thr_bits=int(s[0]), real_n=int(s[1]), num=int(s[2]), t=int(s[3]), gflip=int(s[4]),
                    queue_len=int(s[5]), batch_num=int(s[6]), window=int(s[7]), decay_importance=dec.value,
                    threshold=float(np.array([s[0]], np.uint32).view(np.float32)[0]))

    def stats(self) -> dict:
        s = np.zeros(len(STAT_NAMES), np.int64)
        self.lib.cafe_sketch_stats(self.handle, _np_ptr(s, _lib._i64p))
        return dict(zip(STAT_NAMES, (int(x) for x in s)))

    def state(self) -> dict:
        """Whole state as numpy arrays, in the layout the CPU oracle dumps."""
        sc = self.scalars()
        n1, n2 = self.n1, self.n2
        a = dict(main_val=np.zeros(n1 * 4, np.uint32), main_cnt=np.zeros(n1 * 4, np.float32),
                 main_dic=np.zeros(n1 * 4, np.int32), main_flip=np.zeros(n1, np.uint8),
                 lru_val=np.zeros(n2 * 4, np.uint32), lru_cnt=np.zeros(n2 * 4, np.float32),
                 lru_dic=np.zeros(n2 * 4, np.int32), lru_t=np.zeros(n2 * 4, np.int32), lru_flip=np.zeros(n2, np.uint8),
                 queue=np.zeros(max(sc["queue_len"], 1), np.uint32))
        with torch.cuda.device(self.device):
            _lib.check(self.lib.cafe_sketch_dump(
                self.handle, _np_ptr(a["main_val"], _lib._u32p), _np_ptr(a["main_cnt"], _lib._f32p),
                _np_ptr(a["main_dic"], _lib._i32p), _np_ptr(a["main_flip"], _lib._u8p), _np_ptr(a["lru_val"], _lib._u32p),
                _np_ptr(a["lru_cnt"], _lib._f32p), _np_ptr(a["lru_dic"], _lib._i32p), _np_ptr(a["lru_t"], _lib._i32p),
                _np_ptr(a["lru_flip"], _lib._u8p), _np_ptr(a["queue"], _lib._u32p), _stream()), "cafe_sketch_dump")
        a["queue"] = a["queue"][:sc["queue_len"]].copy()
        a.update(thr_bits=sc["thr_bits"], real_n=sc["real_n"], num=sc["num"], t=sc["t"], gflip=sc["gflip"],
                 batch_num=sc["batch_num"], decay_importance=sc["decay_importance"])
        return a

    def load_state(self, st: dict) -> None:
        """Inverse of state(): restores a sketch saved earlier (same hotn)."""
        c = {k: np.ascontiguousarray(st[k]) for k in _STATE_ARRAYS}
        if c["main_val"].size != self.n1 * 4 or c["lru_val"].size != self.n2 * 4:
            raise ValueError("state was saved from a sketch of another size")
        q = c["queue"].astype(np.uint32)
        qbuf = q if q.size else np.zeros(1, np.uint32)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.cafe_sketch_load(
                self.handle, _np_ptr(c["main_val"].astype(np.uint32), _lib._u32p), _np_ptr(c["main_cnt"].astype(np.float32), _lib._f32p),
                _np_ptr(c["main_dic"].astype(np.int32), _lib._i32p), _np_ptr(c["main_flip"].astype(np.uint8), _lib._u8p),
                _np_ptr(c["lru_val"].astype(np.uint32), _lib._u32p), _np_ptr(c["lru_cnt"].astype(np.float32), _lib._f32p),
                _np_ptr(c["lru_dic"].astype(np.int32), _lib._i32p), _np_ptr(c["lru_t"].astype(np.int32), _lib._i32p),
                _np_ptr(c["lru_flip"].astype(np.uint8), _lib._u8p), _np_ptr(qbuf, _lib._u32p), int(q.size), _stream()),
                "cafe_sketch_load")
        s = np.array([st["thr_bits"], st["real_n"], st["num"], st["t"], st["gflip"], q.size, st["batch_num"], 0], np.int64)
        self.lib.cafe_sketch_set_scalars(self.handle, _np_ptr(s, _lib._i64p), float(st["decay_importance"]))
