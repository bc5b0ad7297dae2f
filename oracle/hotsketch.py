"""ctypes bindings for the CPU oracles.  TEST INFRASTRUCTURE ONLY.

Two interchangeable objects with the same methods:

* ``OracleSketch``    -- the plain-C restatement (oracle/hotsketch_oracle.c), one instance per object;
* ``ReferenceSketch`` -- the reference's own tricks/sketch.cpp compiled by oracle/build_ref.sh
  (process-global state, so at most one live instance per loaded copy of the library).

Nothing in the product package imports this module; tests, the smoke check and the benchmark's CPU
baseline do.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import tempfile
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
ORACLE_SO = _HERE / "_build" / "libhotsketch_oracle.so"
REF_SO = _HERE / "_ref" / "libsketch_ref.so"

_u32p = ctypes.POINTER(ctypes.c_uint32)
_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)
_u8p = ctypes.POINTER(ctypes.c_uint8)
_i64p = ctypes.POINTER(ctypes.c_int64)


def build(force: bool = False) -> None:
    """Compile the C restatement (always) and the patched reference (when its checkout exists)."""
    if force or not ORACLE_SO.exists() or ORACLE_SO.stat().st_mtime < (_HERE / "hotsketch_oracle.c").stat().st_mtime:
        subprocess.run(["make", "-s", "-C", str(_HERE), str(ORACLE_SO)], check=True)
    if force or not REF_SO.exists():
        subprocess.run(["bash", str(_HERE / "build_ref.sh"), str(reference_root())], check=True, stdout=subprocess.DEVNULL)


def _ptr(a: np.ndarray, typ):
    return a.ctypes.data_as(typ)


def _as_ids(ids) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(ids).astype(np.uint32, copy=False))


class OracleSketch:
    """The C restatement.  ``thr`` is converted to float32 like the reference's init does."""

    def __init__(self, lim: int, thr: float, adjust: int = 1, alpha: float = 1.0000005):
        build()
        self._lib = lib = ctypes.CDLL(str(ORACLE_SO))
        lib.hs_new.restype = ctypes.c_void_p
        lib.hs_new.argtypes = [ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_double]
        lib.hs_free.argtypes = [ctypes.c_void_p]
        lib.hs_batch_query.argtypes = [ctypes.c_void_p, _u32p, ctypes.c_int, _i32p]
        lib.hs_batch_insert_val.argtypes = [ctypes.c_void_p, _u32p, _f32p, ctypes.c_int, _i32p]
        lib.hs_reset.argtypes = [ctypes.c_void_p]
        lib.hs_analyse.restype = ctypes.c_double
        lib.hs_analyse.argtypes = [ctypes.c_void_p, _u32p, ctypes.c_int]
        lib.hs_analyse1.restype = ctypes.c_double
        lib.hs_analyse1.argtypes = [ctypes.c_void_p, _u32p, ctypes.c_int]
        lib.hs_n1.argtypes = [ctypes.c_void_p]
        lib.hs_n2.argtypes = [ctypes.c_void_p]
        lib.hs_scalars.argtypes = [ctypes.c_void_p, _i64p, ctypes.POINTER(ctypes.c_double)]
        lib.hs_counters.argtypes = [ctypes.c_void_p, _i64p]
        lib.hs_dump_main.argtypes = [ctypes.c_void_p, _u32p, _f32p, _i32p, _u8p]
        lib.hs_dump_lru.argtypes = [ctypes.c_void_p, _u32p, _f32p, _i32p, _i32p, _u8p]
        lib.hs_dump_queue.restype = ctypes.c_int64
        lib.hs_dump_queue.argtypes = [ctypes.c_void_p, _u32p]
        self._h = lib.hs_new(int(lim), float(thr), int(adjust), float(alpha))
        self.lim = int(lim)
        self.n1 = lib.hs_n1(self._h)
        self.n2 = lib.hs_n2(self._h)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.hs_free(self._h)
            self._h = None

    def batch_query(self, ids) -> np.ndarray:
        ids = _as_ids(ids)
        out = np.empty(ids.size, np.int32)
        self._lib.hs_batch_query(self._h, _ptr(ids, _u32p), ids.size, _ptr(out, _i32p))
        return out

    def batch_insert_val(self, ids, v=None) -> np.ndarray:
        ids = _as_ids(ids)
        out = np.empty(ids.size, np.int32)
        vp = None
        if v is not None:
            v = np.ascontiguousarray(v, np.float32)
            assert v.size == ids.size
            vp = _ptr(v, _f32p)
        self._lib.hs_batch_insert_val(self._h, _ptr(ids, _u32p), vp, ids.size, _ptr(out, _i32p))
        return out

    def batch_insert(self, ids) -> np.ndarray:
        return self.batch_insert_val(ids, None)

    def reset(self) -> None:
        self._lib.hs_reset(self._h)

    def analyse(self, ids) -> float:
        ids = _as_ids(ids)
        return self._lib.hs_analyse(self._h, _ptr(ids, _u32p), ids.size)

    def analyse1(self, ids) -> float:
        ids = _as_ids(ids)
        return self._lib.hs_analyse1(self._h, _ptr(ids, _u32p), ids.size)

    def counters(self) -> dict:
        c = np.zeros(9, np.int64)
        self._lib.hs_counters(self._h, _ptr(c, _i64p))
        names = ["main_hit", "lru_hit", "lru_new", "promote_own", "promote_victim", "insert_fail",
                 "resets", "resets_refused", "flips"]
        return dict(zip(names, (int(x) for x in c)))

    def state(self) -> dict:
        """Full state as numpy arrays, in the layout every implementation dumps to."""
        n1, n2 = self.n1, self.n2
        s = np.zeros(8, np.int64)
        dec = ctypes.c_double()
        self._lib.hs_scalars(self._h, _ptr(s, _i64p), ctypes.byref(dec))
        mv, mc, md, mf = np.zeros(n1 * 4, np.uint32), np.zeros(n1 * 4, np.float32), np.zeros(n1 * 4, np.int32), np.zeros(n1, np.uint8)
        self._lib.hs_dump_main(self._h, _ptr(mv, _u32p), _ptr(mc, _f32p), _ptr(md, _i32p), _ptr(mf, _u8p))
        lv, lc, ld, lt, lf = (np.zeros(n2 * 4, np.uint32), np.zeros(n2 * 4, np.float32), np.zeros(n2 * 4, np.int32),
                              np.zeros(n2 * 4, np.int32), np.zeros(n2, np.uint8))
        self._lib.hs_dump_lru(self._h, _ptr(lv, _u32p), _ptr(lc, _f32p), _ptr(ld, _i32p), _ptr(lt, _i32p), _ptr(lf, _u8p))
        qn = self._lib.hs_dump_queue(self._h, None)
        q = np.zeros(max(qn, 1), np.uint32)
        self._lib.hs_dump_queue(self._h, _ptr(q, _u32p))
        return dict(thr_bits=int(s[0]), real_n=int(s[1]), num=int(s[2]), t=int(s[3]), gflip=int(s[4]),
                    batch_num=int(s[6]), decay_importance=dec.value,
                    main_val=mv, main_cnt=mc, main_dic=md, main_flip=mf,
                    lru_val=lv, lru_cnt=lc, lru_dic=ld, lru_t=lt, lru_flip=lf, queue=q[:qn].copy())


class _MutedStdout:
    """The reference prints progress lines from C; keep them out of the caller's stdout."""

    def __enter__(self):
        import sys
        sys.stdout.flush()
        self._saved = os.dup(1)
        self._null = os.open(os.devnull, os.O_WRONLY)
        os.dup2(self._null, 1)

    def __exit__(self, *exc):
        # flush the C library's buffer into the null device before restoring
        ctypes.CDLL(None).fflush(None)
        os.dup2(self._saved, 1)
        os.close(self._saved)
        os.close(self._null)


def reference_root() -> Path:
    """Where the reference checkout is looked for: $CAFE_REFERENCE_ROOT, else a directory named
    `reference` beside this repository."""
    env = os.environ.get("CAFE_REFERENCE_ROOT")
    return Path(env) if env else _HERE.parent.parent / "reference"


def ref_available() -> bool:
    if not REF_SO.exists() and (reference_root() / "tricks" / "sketch.cpp").exists():
        build()
    return REF_SO.exists()


class ReferenceSketch:
    """The compiled reference.  Its state is process-global, so a process's first instance loads
    oracle/_ref/libsketch_ref.so itself and every further one a private temp-file copy of it, which
    gives independent sketches in one process."""

    _direct_used = False

    def __init__(self, lim: int, thr: float, adjust: int = 1, alpha: float = 1.0000005):
        if not ref_available():
            raise RuntimeError("oracle/_ref/libsketch_ref.so has not been built (reference checkout absent)")
        if not ReferenceSketch._direct_used:
            ReferenceSketch._direct_used = True
            self._lib = lib = ctypes.CDLL(str(REF_SO))
        else:
            fd, self._tmp = tempfile.mkstemp(suffix=".so", prefix="sketch_ref_")
            os.close(fd)
            shutil.copyfile(REF_SO, self._tmp)
            self._lib = lib = ctypes.CDLL(self._tmp)
            os.unlink(self._tmp)
        lib.init.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_double]
        lib.init.restype = None
        for name in ("batch_query", "batch_insert"):
            f = getattr(lib, name)
            f.argtypes = [_u32p, ctypes.c_int]
            f.restype = _i32p
        lib.batch_insert_val.argtypes = [_u32p, _f32p, ctypes.c_int]
        lib.batch_insert_val.restype = _i32p
        for name in ("analyse", "analyse1"):
            f = getattr(lib, name)
            f.argtypes = [_u32p, ctypes.c_int]
            f.restype = ctypes.c_double
        lib.ref_scalars.argtypes = [_i64p, ctypes.POINTER(ctypes.c_double)]
        lib.ref_dump_main.argtypes = [_u32p, _f32p, _i32p, _u8p]
        lib.ref_dump_lru.argtypes = [_u32p, _f32p, _i32p, _i32p, _u8p]
        lib.ref_dump_queue.restype = ctypes.c_int64
        lib.ref_dump_queue.argtypes = [_u32p]
        if float(thr) != int(thr):
            raise ValueError("the reference's init() takes an integer threshold")
        with _MutedStdout():
            lib.ref_reset_globals()
            lib.init(int(lim), int(thr), int(adjust), float(alpha))
        self.lim = int(lim)
        self.n1 = lib.ref_n1()
        self.n2 = lib.ref_n2()

    MAX_N = 1 << 22

    def _out(self, p, n) -> np.ndarray:
        return np.ctypeslib.as_array(p, shape=(n,)).copy()

    def batch_query(self, ids) -> np.ndarray:
        ids = _as_ids(ids)
        assert ids.size <= self.MAX_N
        return self._out(self._lib.batch_query(_ptr(ids, _u32p), ids.size), ids.size)

    def batch_insert_val(self, ids, v=None) -> np.ndarray:
        ids = _as_ids(ids)
        assert ids.size <= self.MAX_N
        with _MutedStdout():
            if v is None:
                p = self._lib.batch_insert(_ptr(ids, _u32p), ids.size)
            else:
                v = np.ascontiguousarray(v, np.float32)
                p = self._lib.batch_insert_val(_ptr(ids, _u32p), _ptr(v, _f32p), ids.size)
        return self._out(p, ids.size)

    def batch_insert(self, ids) -> np.ndarray:
        return self.batch_insert_val(ids, None)

    def analyse(self, ids) -> float:
        ids = _as_ids(ids)
        return self._lib.analyse(_ptr(ids, _u32p), ids.size)

    def analyse1(self, ids) -> float:
        ids = _as_ids(ids)
        return self._lib.analyse1(_ptr(ids, _u32p), ids.size)

    def state(self) -> dict:
        n1, n2 = self.n1, self.n2
        s = np.zeros(8, np.int64)
        dec = ctypes.c_double()
        self._lib.ref_scalars(_ptr(s, _i64p), ctypes.byref(dec))
        mv, mc, md, mf = np.zeros(n1 * 4, np.uint32), np.zeros(n1 * 4, np.float32), np.zeros(n1 * 4, np.int32), np.zeros(n1, np.uint8)
        self._lib.ref_dump_main(_ptr(mv, _u32p), _ptr(mc, _f32p), _ptr(md, _i32p), _ptr(mf, _u8p))
        lv, lc, ld, lt, lf = (np.zeros(n2 * 4, np.uint32), np.zeros(n2 * 4, np.float32), np.zeros(n2 * 4, np.int32),
                              np.zeros(n2 * 4, np.int32), np.zeros(n2, np.uint8))
        self._lib.ref_dump_lru(_ptr(lv, _u32p), _ptr(lc, _f32p), _ptr(ld, _i32p), _ptr(lt, _i32p), _ptr(lf, _u8p))
        qn = self._lib.ref_dump_queue(None)
        q = np.zeros(max(qn, 1), np.uint32)
        self._lib.ref_dump_queue(_ptr(q, _u32p))
        return dict(thr_bits=int(s[0]), real_n=int(s[1]), num=int(s[2]), t=int(s[3]), gflip=int(s[4]),
                    batch_num=int(s[6]), decay_importance=dec.value,
                    main_val=mv, main_cnt=mc, main_dic=md, main_flip=mf,
                    lru_val=lv, lru_cnt=lc, lru_dic=ld, lru_t=lt, lru_flip=lf, queue=q[:qn].copy())


def states_equal(a: dict, b: dict) -> list[str]:
    """Names of the state fields that differ (empty list = bit-identical states)."""
    bad = []
    for k in a:
        if isinstance(a[k], np.ndarray):
            x, y = a[k], b[k]
            if x.dtype == np.float32:
                x, y = x.view(np.uint32), y.view(np.uint32)
            if x.shape != y.shape or not np.array_equal(x, y):
                bad.append(k)
        elif a[k] != b[k]:
            bad.append(k)
    return bad
