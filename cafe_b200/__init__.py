"""cafe_b200: the CAFE compressed-embedding hot path (HotSketch + SKEmbeddingBag) on B200 CUDA kernels.

Importing the package loads libcafe_b200.so; it raises if the library has not been built
(`python -m cafe_b200.build`).  There is no CPU path.
"""
from . import _lib, sizing
from ._lib import CafeError, INSERT_PARALLEL, INSERT_SEQUENTIAL

_lib.load()

from .sketch import HotSketch  # noqa: E402
from .sk_embedding_bag import SKEmbeddingBag, SKEmbeddingGroup, attach_optimizer  # noqa: E402

__all__ = ["HotSketch", "SKEmbeddingBag", "SKEmbeddingGroup", "attach_optimizer", "sizing", "CafeError",
           "INSERT_PARALLEL", "INSERT_SEQUENTIAL", "load_library"]


def load_library():
    """The ctypes library object; pass it where the reference's code expects `lib` (it exports init,
    batch_query, batch_insert, batch_insert_val, analyse, analyse1 like the reference's sklib.so)."""
    return _lib.load()
