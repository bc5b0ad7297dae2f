"""Per-kernel timing of the library's own launches (CUDA events on the launching stream) and launch counts."""
from __future__ import annotations

import ctypes

import numpy as np

from . import _lib


def slot_names() -> list[str]:
    lib = _lib.load()
    return [lib.cafe_profile_slot_name(i).decode() for i in range(lib.cafe_profile_slots())]


def enable(on: bool = True) -> None:
    _lib.load().cafe_profile_enable(1 if on else 0)


def read() -> dict:
    """{slot: (ms, launches)} since the last read; synchronises the device."""
    lib = _lib.load()
    n = lib.cafe_profile_slots()
    ms = np.zeros(n, np.float64)
    cnt = np.zeros(n, np.int64)
    _lib.check(lib.cafe_profile_read(ms.ctypes.data_as(ctypes.POINTER(ctypes.c_double)),
                                     cnt.ctypes.data_as(_lib._i64p)), "cafe_profile_read")
    return {name: (float(ms[i]), int(cnt[i])) for i, name in enumerate(slot_names())}


def launch_count() -> int:
    return int(_lib.load().cafe_launch_count())
