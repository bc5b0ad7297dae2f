"""ctypes bindings for the CPU oracles of the one-stage HotSketch.  TEST INFRASTRUCTURE ONLY.

``OracleSigmod``    -- the plain-C restatement (oracle/sigmod_oracle.c), one instance per object;
``ReferenceSigmod`` -- the reference's own ArtifactEvaluation/embeddings/sketch.cpp compiled by
                       oracle/build_ref.sh (its sketches live in a file-scope array; this class uses number 0, so a
                       process's first instance loads the library itself and further ones a private copy).
Nothing in the product package imports this module.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import tempfile
from pathlib import Path

import numpy as np

from .hotsketch import _MutedStdout, reference_root

_HERE = Path(__file__).resolve().parent
ORACLE_SO = _HERE / "_build" / "libsigmod_oracle.so"
REF_SO = _HERE / "_ref" / "libsketch_sigmod_ref.so"
_u32p, _i32p, _f32p, _i64p = (ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_float),
                              ctypes.POINTER(ctypes.c_int64))


def build(force: bool = False) -> None:
    src = _HERE / "sigmod_oracle.c"
    if force or not ORACLE_SO.exists() or ORACLE_SO.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-s", "-C", str(_HERE), str(ORACLE_SO)], check=True)
    if (force or not REF_SO.exists()) and (reference_root() / "ArtifactEvaluation" / "embeddings" / "sketch.cpp").exists():
        subprocess.run(["bash", str(_HERE / "build_ref.sh"), str(reference_root())], check=True, stdout=subprocess.DEVNULL)


def ref_available() -> bool:
    if not REF_SO.exists():
        build()
    return REF_SO.exists()


def _ids(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a).astype(np.uint32, copy=False))


class OracleSigmod:
    def __init__(self, lim: int, k: int, decay_rate: float = 0.99):
        build()
        self._lib = lib = ctypes.CDLL(str(ORACLE_SO))
        lib.sg_new.restype = ctypes.c_void_p
        lib.sg_new.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_double]
        lib.sg_free.argtypes = [ctypes.c_void_p]
        lib.sg_batch_query.argtypes = [ctypes.c_void_p, _u32p, ctypes.c_int, _i32p]
        lib.sg_batch_insert_val.argtypes = [ctypes.c_void_p, _u32p, _f32p, ctypes.c_int, _i32p]
        lib.sg_update.argtypes = [ctypes.c_void_p]
        lib.sg_scalars.argtypes = [ctypes.c_void_p, _i64p, ctypes.POINTER(ctypes.c_double)]
        lib.sg_dump.argtypes = [ctypes.c_void_p, _u32p, _f32p, _i32p, _u32p]
        self._h = lib.sg_new(int(k), int(lim), float(decay_rate))
        self.lim, self.k = int(lim), int(k)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.sg_free(self._h)
            self._h = None

    def batch_query(self, ids) -> np.ndarray:
        ids = _ids(ids)
        out = np.empty(ids.size, np.int32)
        self._lib.sg_batch_query(self._h, ids.ctypes.data_as(_u32p), ids.size, out.ctypes.data_as(_i32p))
        return out

    def batch_insert_val(self, ids, v=None) -> np.ndarray:
        ids = _ids(ids)
        out = np.empty(ids.size, np.int32)
        vp = None
        if v is not None:
            v = np.ascontiguousarray(v, np.float32)
            vp = v.ctypes.data_as(_f32p)
        self._lib.sg_batch_insert_val(self._h, ids.ctypes.data_as(_u32p), vp, ids.size, out.ctypes.data_as(_i32p))
        return out

    def batch_insert(self, ids) -> np.ndarray:
        return self.batch_insert_val(ids, None)

    def update(self) -> None:
        self._lib.sg_update(self._h)

    def state(self) -> dict:
        s = np.zeros(5, np.int64)
        tot = ctypes.c_double()
        self._lib.sg_scalars(self._h, s.ctypes.data_as(_i64p), ctypes.byref(tot))
        n = self.lim
        val, cnt, dic = np.zeros(n * 4, np.uint32), np.zeros(n * 4, np.float32), np.zeros(n * 4, np.int32)
        q = np.zeros(max(int(s[1]), 1), np.uint32)
        self._lib.sg_dump(self._h, val.ctypes.data_as(_u32p), cnt.ctypes.data_as(_f32p), dic.ctypes.data_as(_i32p),
                          q.ctypes.data_as(_u32p))
        return dict(num=int(s[0]), tot=tot.value, val=val, cnt=cnt, dic=dic, queue=q[:int(s[1])].copy())


class ReferenceSigmod:
    _direct_used = False

    def __init__(self, lim: int, k: int, decay_rate: float = 0.99):
        if not ref_available():
            raise RuntimeError("oracle/_ref/libsketch_sigmod_ref.so has not been built (reference checkout absent)")
        if not ReferenceSigmod._direct_used:
            ReferenceSigmod._direct_used = True
            self._lib = lib = ctypes.CDLL(str(REF_SO))
        else:
            fd, tmp = tempfile.mkstemp(suffix=".so", prefix="sketch_sigmod_ref_")
            os.close(fd)
            shutil.copyfile(REF_SO, tmp)
            self._lib = lib = ctypes.CDLL(tmp)
            os.unlink(tmp)
        lib.init.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_double, ctypes.c_int]
        lib.init.restype = None
        for name in ("batch_query", "batch_insert"):
            f = getattr(lib, name)
            f.argtypes = [_u32p, ctypes.c_int, ctypes.c_int]
            f.restype = _i32p
        lib.batch_insert_val.argtypes = [_u32p, _f32p, ctypes.c_int, ctypes.c_int]
        lib.batch_insert_val.restype = _i32p
        lib.refsg_scalars.argtypes = [_i64p, ctypes.POINTER(ctypes.c_double)]
        lib.refsg_dump.argtypes = [_u32p, _f32p, _i32p, _u32p]
        with _MutedStdout():
            lib.init(int(lim), int(k), float(decay_rate), 0)
        self.lim, self.k = int(lim), int(k)

    def batch_query(self, ids) -> np.ndarray:
        ids = _ids(ids)
        return np.ctypeslib.as_array(self._lib.batch_query(ids.ctypes.data_as(_u32p), ids.size, 0), shape=(ids.size,)).copy()

    def batch_insert_val(self, ids, v=None) -> np.ndarray:
        ids = _ids(ids)
        with _MutedStdout():
            if v is None:
                p = self._lib.batch_insert(ids.ctypes.data_as(_u32p), ids.size, 0)
            else:
                v = np.ascontiguousarray(v, np.float32)
                p = self._lib.batch_insert_val(ids.ctypes.data_as(_u32p), v.ctypes.data_as(_f32p), ids.size, 0)
        return np.ctypeslib.as_array(p, shape=(ids.size,)).copy()

    def batch_insert(self, ids) -> np.ndarray:
        return self.batch_insert_val(ids, None)

    def state(self) -> dict:
        s = np.zeros(5, np.int64)
        tot = ctypes.c_double()
        self._lib.refsg_scalars(s.ctypes.data_as(_i64p), ctypes.byref(tot))
        n = self.lim
        val, cnt, dic = np.zeros(n * 4, np.uint32), np.zeros(n * 4, np.float32), np.zeros(n * 4, np.int32)
        q = np.zeros(max(int(s[1]), 1), np.uint32)
        self._lib.refsg_dump(val.ctypes.data_as(_u32p), cnt.ctypes.data_as(_f32p), dic.ctypes.data_as(_i32p),
                             q.ctypes.data_as(_u32p))
        return dict(num=int(s[0]), tot=tot.value, val=val, cnt=cnt, dic=dic, queue=q[:int(s[1])].copy())
