"""CPU emulation of the device sketch engine (tests only): builds hostemu.cpp and binds it."""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "_build" / "libcafe_hostemu.so"
_CSRC = _HERE.parent.parent / "cafe_b200" / "csrc"

_u32p = ctypes.POINTER(ctypes.c_uint32)
_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)
_u8p = ctypes.POINTER(ctypes.c_uint8)
_i64p = ctypes.POINTER(ctypes.c_int64)

STAT_NAMES = ["calls", "lookups", "rounds", "jobs", "truncated_jobs", "resets", "resets_refused", "flips",
              "seq_fallbacks", "main_hits", "lru_visits", "events", "max_rounds"]


def build() -> Path:
    srcs = [_HERE / "hostemu.cpp", _CSRC / "sketch_core.cuh", _CSRC / "sketch_engine.h", _CSRC / "cafe_types.h"]
    if not _SO.exists() or _SO.stat().st_mtime < max(s.stat().st_mtime for s in srcs):
        _SO.parent.mkdir(exist_ok=True)
        subprocess.run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-x", "c++",
                        str(_HERE / "hostemu.cpp"), "-o", str(_SO)], check=True)
    return _SO


def _p(a, t):
    return a.ctypes.data_as(t)


class EmuSketch:
    def __init__(self, lim, thr, adjust=1, alpha=1.0000005, cap=1 << 20, parallel=True):
        self._lib = lib = ctypes.CDLL(str(build()))
        lib.emu_new.restype = ctypes.c_void_p
        lib.emu_new.argtypes = [ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_double, ctypes.c_int]
        lib.emu_free.argtypes = [ctypes.c_void_p]
        lib.emu_n1.argtypes = [ctypes.c_void_p]
        lib.emu_n2.argtypes = [ctypes.c_void_p]
        lib.emu_query.argtypes = [ctypes.c_void_p, _u32p, ctypes.c_int, _i32p]
        lib.emu_insert.argtypes = [ctypes.c_void_p, _u32p, _f32p, _i32p, ctypes.c_int, _i32p, _i32p, ctypes.c_int]
        lib.emu_refit.argtypes = [ctypes.c_void_p]
        lib.emu_set_window.argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib.emu_set_round_cap.argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib.emu_set_job_sizing.argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib.emu_scalars.argtypes = [ctypes.c_void_p, _i64p, ctypes.POINTER(ctypes.c_double)]
        lib.emu_stats.argtypes = [ctypes.c_void_p, _i64p]
        lib.emu_dump.argtypes = [ctypes.c_void_p, _u32p, _f32p, _i32p, _u8p, _u32p, _f32p, _i32p, _i32p, _u8p, _u32p]
        self._h = lib.emu_new(int(lim), float(thr), int(adjust), float(alpha), int(cap))
        assert self._h
        self.n1, self.n2 = lib.emu_n1(self._h), lib.emu_n2(self._h)
        self.parallel = parallel
        self.last_post_row = None

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.emu_free(self._h)
            self._h = None

    def batch_query(self, ids):
        ids = np.ascontiguousarray(np.asarray(ids).astype(np.uint32, copy=False))
        out = np.empty(ids.size, np.int32)
        assert self._lib.emu_query(self._h, _p(ids, _u32p), ids.size, _p(out, _i32p)) == 0
        return out

    def insert_segments(self, ids, v, seg_off, want_post=True):
        ids = np.ascontiguousarray(np.asarray(ids).astype(np.uint32, copy=False))
        seg = np.ascontiguousarray(seg_off, np.int32)
        mask = np.zeros(ids.size, np.int32)
        post = np.zeros(ids.size, np.int32) if want_post else None
        vp = None
        if v is not None:
            v = np.ascontiguousarray(v, np.float32)
            vp = _p(v, _f32p)
        rc = self._lib.emu_insert(self._h, _p(ids, _u32p), vp, _p(seg, _i32p), seg.size - 1, _p(mask, _i32p),
                                  _p(post, _i32p) if want_post else None, 1 if self.parallel else 0)
        self.last_rc = rc
        self.last_post_row = post
        return mask

    def batch_insert_val(self, ids, v=None):
        return self.insert_segments(ids, v, [0, len(ids)])

    def set_window(self, w):
        self._lib.emu_set_window(self._h, w)

    def set_round_cap(self, c):
        self._lib.emu_set_round_cap(self._h, c)

    def set_job_sizing(self, by_rate):
        self._lib.emu_set_job_sizing(self._h, 1 if by_rate else 0)

    def refit(self):
        return self._lib.emu_refit(self._h)

    def stats(self):
        s = np.zeros(len(STAT_NAMES), np.int64)
        self._lib.emu_stats(self._h, _p(s, _i64p))
        return dict(zip(STAT_NAMES, (int(x) for x in s)))

    def state(self):
        n1, n2 = self.n1, self.n2
        s = np.zeros(8, np.int64)
        dec = ctypes.c_double()
        self._lib.emu_scalars(self._h, _p(s, _i64p), ctypes.byref(dec))
        mv, mc, md, mf = np.zeros(n1 * 4, np.uint32), np.zeros(n1 * 4, np.float32), np.zeros(n1 * 4, np.int32), np.zeros(n1, np.uint8)
        lv, lc, ld, lt, lf = (np.zeros(n2 * 4, np.uint32), np.zeros(n2 * 4, np.float32), np.zeros(n2 * 4, np.int32),
                              np.zeros(n2 * 4, np.int32), np.zeros(n2, np.uint8))
        q = np.zeros(max(int(s[5]), 1), np.uint32)
        self._lib.emu_dump(self._h, _p(mv, _u32p), _p(mc, _f32p), _p(md, _i32p), _p(mf, _u8p), _p(lv, _u32p),
                           _p(lc, _f32p), _p(ld, _i32p), _p(lt, _i32p), _p(lf, _u8p), _p(q, _u32p))
        return dict(thr_bits=int(s[0]), real_n=int(s[1]), num=int(s[2]), t=int(s[3]), gflip=int(s[4]),
                    batch_num=int(s[6]), decay_importance=dec.value,
                    main_val=mv, main_cnt=mc, main_dic=md, main_flip=mf,
                    lru_val=lv, lru_cnt=lc, lru_dic=ld, lru_t=lt, lru_flip=lf, queue=q[:int(s[5])].copy())
