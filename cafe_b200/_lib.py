"""Loads libcafe_b200.so (the C-ABI library of include/cafe_b200.h) and declares its signatures.

There is no fallback: if the library has not been built, importing the package fails with the build
command in the message.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_uint8, c_uint32, c_void_p
from pathlib import Path

_PKG = Path(__file__).resolve().parent
SO_PATH = _PKG / "libcafe_b200.so"

OK, ERR_ARG, ERR_CAPACITY, ERR_CUDA, ERR_NOCONVERGE, ERR_RESET_UNDERFLOW, ERR_UNSUPPORTED = range(7)
INSERT_PARALLEL, INSERT_SEQUENTIAL = 0, 1
MAX_FIELDS = 64
_STATUS_NAMES = {ERR_ARG: "invalid argument", ERR_CAPACITY: "capacity exceeded", ERR_CUDA: "CUDA error",
                 ERR_NOCONVERGE: "parallel insert did not converge (sequential kernel used)",
                 ERR_RESET_UNDERFLOW: "threshold re-fit refused", ERR_UNSUPPORTED: "unsupported shape"}
# statuses that report something but leave exact results
INFORMATIONAL = (ERR_NOCONVERGE, ERR_RESET_UNDERFLOW)

_vp = c_void_p
_u32p, _i32p, _f32p, _u8p, _i64p = (POINTER(c_uint32), POINTER(c_int32), POINTER(c_float), POINTER(c_uint8),
                                    POINTER(c_int64))

# name -> (restype, argtypes); every symbol include/cafe_b200.h declares
SIGNATURES = {
    "cafe_last_error": (c_char_p, []),
    "cafe_sketch_create": (c_int, [POINTER(_vp), c_int, c_float, c_int, c_double, c_int]),
    "cafe_sketch_destroy": (c_int, [_vp]),
    "cafe_sketch_query": (c_int, [_vp, _vp, c_int, _vp, _vp]),
    "cafe_sketch_insert": (c_int, [_vp, _vp, _vp, POINTER(c_int), c_int, _vp, _vp, c_int, _vp]),
    "cafe_sketch_refit": (c_int, [_vp, _vp]),
    "cafe_sketch_sizes": (c_int, [_vp, POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_int)]),
    "cafe_sketch_scalars": (c_int, [_vp, _i64p, POINTER(c_double)]),
    "cafe_sketch_set_scalars": (c_int, [_vp, _i64p, c_double]),
    "cafe_sketch_tuning": (c_int, [_vp, c_int, c_int]),
    "cafe_sketch_stats": (c_int, [_vp, _i64p]),
    "cafe_sketch_dump": (c_int, [_vp, _u32p, _f32p, _i32p, _u8p, _u32p, _f32p, _i32p, _i32p, _u8p, _u32p, _vp]),
    "cafe_sketch_load": (c_int, [_vp, _u32p, _f32p, _i32p, _u8p, _u32p, _f32p, _i32p, _i32p, _u8p, _u32p, c_int, _vp]),
    "cafe_embed_forward": (c_int, [_vp, _vp, c_int, c_int, c_int, _i64p, _i32p, POINTER(_vp), _vp, c_int, c_int, _vp,
                                   c_int64, c_int64, _vp, _vp, _vp]),
    "cafe_records_to_batch": (c_int, [_vp, c_int, c_int, _vp, c_int, _vp, _vp, _vp]),
    "cafe_embed_resolve": (c_int, [_vp, _vp, c_int, c_int, c_int, _i64p, _i32p, c_int, _vp, _vp, _vp]),
    "cafe_embed_gather": (c_int, [_vp, _vp, c_int, c_int, _i32p, POINTER(_vp), _vp, c_int, c_int, _vp, c_int64, c_int64, _vp]),
    "cafe_embed_gather_sharded": (c_int, [_vp, _vp, c_int, c_int, _i32p, POINTER(_vp), _vp, c_int, c_int, POINTER(_vp), c_int,
                                          c_int, c_int64, c_int64, _vp]),
    "cafe_grad_importance": (c_int, [_vp, _vp, c_int64, c_int64, c_int, c_int, c_int, _vp, _vp]),
    "cafe_grad_importance_static": (c_int, [_vp, c_int64, c_int64, c_int, c_int, c_int, _vp, _vp]),
    "cafe_migrate": (c_int, [_vp, _vp, c_int, _vp, _vp, c_int, c_int, _i64p, _i32p, POINTER(_vp), _vp, c_int, c_int,
                             _vp, _vp]),
    "cafe_scatter_sgd": (c_int, [_vp, _vp, c_int64, c_int64, _vp, c_int, c_int, _i32p, POINTER(_vp), _vp, c_int, c_int,
                                 c_float, _vp]),
    "cafe_embed_backward": (c_int, [_vp, _vp, c_int64, c_int64, _vp, c_int, _vp, _vp, c_int, c_int, _i64p, _i32p,
                                    POINTER(_vp), _vp, c_int, c_int, c_float, c_int, _vp, _vp, _vp]),
    "cafe_embed_backward_begin": (c_int, [_vp, _vp, _vp, c_int, c_int, _i32p, POINTER(_vp), _vp, c_int, c_int, c_int, _vp]),
    "cafe_shard_scatter_ids": (c_int, [_vp, c_int, c_int, c_int, c_int, POINTER(_vp), _vp]),
    "cafe_embed_forward_sharded": (c_int, [_vp, _vp, c_int, c_int, c_int, _i64p, _i32p, POINTER(_vp), _vp, c_int, c_int,
                                           POINTER(_vp), c_int, c_int, c_int64, c_int64, _vp, _vp, _vp]),
    "cafe_shard_pull_importance": (c_int, [_vp, POINTER(_vp), c_int, c_int, c_int, c_int, c_int64, c_int64, _vp, _vp, _vp]),
    "cafe_shard_push_grads": (c_int, [_vp, c_int, c_int, c_int, c_int, c_int, POINTER(_vp), _vp]),
    "cafe_shard_push_grads_fields": (c_int, [_vp, c_int, c_int, c_int, c_int, c_int, POINTER(_vp), c_int, c_int, _vp]),
    "cafe_embed_backward_gated": (c_int, [_vp, _vp, c_int64, c_int64, _vp, c_int, _vp, _vp, c_int, c_int, _i64p, _i32p,
                                          POINTER(_vp), _vp, c_int, c_int, c_float, c_int, c_int, _vp, _vp]),
    "cafe_shard_push_norms": (c_int, [_vp, c_int, c_int, c_int, c_int, c_int, POINTER(_vp), _vp, _vp]),
    "cafe_embed_backward_norms": (c_int, [_vp, _vp, c_int64, c_int64, _vp, _vp, c_int, _vp, _vp, c_int, c_int, _i64p, _i32p,
                                          POINTER(_vp), _vp, c_int, c_int, c_float, c_int, _vp, _vp]),
    "cafe_embed_backward_imp": (c_int, [_vp, _vp, c_int64, c_int64, _vp, _vp, c_int, _vp, _vp, c_int, c_int, _i64p, _i32p,
                                        POINTER(_vp), _vp, c_int, c_int, c_float, c_int, _vp, _vp]),
    "cafe_dot_interaction_forward": (c_int, [_vp, _vp, c_int64, c_int64, c_int, c_int, c_int, c_int, _vp, c_int64, _vp]),
    "cafe_dot_interaction_backward": (c_int, [_vp, _vp, c_int64, c_int64, c_int, c_int, c_int, c_int, _vp, c_int64, _vp, _vp,
                                              c_int64, c_int64, _vp]),
    "cafe_sigmod_create": (c_int, [POINTER(_vp), c_int, c_int, c_double, c_int]),
    "cafe_sigmod_destroy": (c_int, [_vp]),
    "cafe_sigmod_query": (c_int, [_vp, _vp, c_int, _vp, _vp]),
    "cafe_sigmod_insert": (c_int, [_vp, _vp, _vp, c_int, _vp, _vp]),
    "cafe_sigmod_update": (c_int, [_vp, _vp]),
    "cafe_sigmod_resolve": (c_int, [_vp, _vp, c_int, c_int64, c_int, c_int, _vp, _vp, _vp]),
    "cafe_sigmod_post_rows": (c_int, [_vp, _vp, _vp, c_int, _vp, _vp]),
    "cafe_sigmod_dump": (c_int, [_vp, _u32p, _f32p, _i32p, _u32p, _i64p, POINTER(c_double), _vp]),
    "cafe_sigmod_load": (c_int, [_vp, _u32p, _f32p, _i32p, c_int64, c_double, _vp]),
    "cafe_workspace_create": (c_int, [POINTER(_vp), c_int, c_int]),
    "cafe_profile_slots": (c_int, []),
    "cafe_profile_slot_name": (c_char_p, [c_int]),
    "cafe_profile_enable": (c_int, [c_int]),
    "cafe_profile_read": (c_int, [POINTER(c_double), _i64p]),
    "cafe_launch_count": (c_int64, []),
    "init": (None, [c_int, c_int, c_int, c_double]),
    "batch_query": (_i32p, [_u32p, c_int]),
    "batch_insert": (_i32p, [_u32p, c_int]),
    "batch_insert_val": (_i32p, [_u32p, _f32p, c_int]),
    "analyse": (c_double, [_u32p, c_int]),
    "analyse1": (c_double, [_u32p, c_int]),
    "cafe_global_handle": (_vp, []),
    "cafe_global_set_capacity": (c_int, [c_int]),
}

_lib = None


def load() -> ctypes.CDLL:
    """The loaded library, with argtypes set.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not SO_PATH.exists():
            raise RuntimeError(
                f"{SO_PATH} is missing: the CUDA library has not been built. Run `python -m cafe_b200.build` "
                "(needs nvcc); there is no CPU fallback.")
        lib = ctypes.CDLL(str(SO_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class CafeError(RuntimeError):
    def __init__(self, status: int, where: str):
        msg = _STATUS_NAMES.get(status, f"status {status}")
        if status == ERR_CUDA:
            msg += ": " + (load().cafe_last_error() or b"").decode(errors="replace")
        super().__init__(f"{where}: {msg}")
        self.status = status


def check(status: int, where: str) -> int:
    """Raises on hard errors; returns informational statuses to the caller."""
    if status == OK or status in INFORMATIONAL:
        return status
    raise CafeError(status, where)
