"""cafe_b200: the CAFE compressed-embedding hot path (HotSketch + SKEmbeddingBag) on B200 CUDA kernels.

Everything here runs on libcafe_b200.so (built by `python -m cafe_b200.build`).  The library is loaded
the first time any name of the package is used; if it is missing that use raises with the build
command in the message.  There is no CPU path.
"""
from __future__ import annotations

__all__ = ["HotSketch", "SKEmbeddingBag", "SKEmbeddingGroup", "attach_optimizer", "sizing", "synthetic", "CafeError",
           "INSERT_PARALLEL", "INSERT_SEQUENTIAL", "load_library", "profile", "SigmodSketch", "SigmodSKEmbeddingBag",
           "dlrm_harness", "sharded"]

INSERT_PARALLEL, INSERT_SEQUENTIAL = 0, 1


def load_library():
    """The ctypes library object; pass it where the reference's code expects `lib` (it exports init,
    batch_query, batch_insert, batch_insert_val, analyse, analyse1 like the reference's sklib.so)."""
    from . import _lib
    return _lib.load()


def __getattr__(name):
    if name in ("HotSketch",):
        load_library()
        from .sketch import HotSketch
        return HotSketch
    if name in ("SKEmbeddingBag", "SKEmbeddingGroup", "attach_optimizer"):
        load_library()
        from . import sk_embedding_bag
        return getattr(sk_embedding_bag, name)
    if name in ("SigmodSketch", "SigmodSKEmbeddingBag"):
        load_library()
        from . import sigmod
        return getattr(sigmod, name)
    if name == "CafeError":
        from ._lib import CafeError
        return CafeError
    if name in ("sizing", "synthetic", "profile", "sharded", "dlrm_harness", "sigmod"):
        import importlib
        return importlib.import_module(f".{name}", __name__)
    raise AttributeError(f"module 'cafe_b200' has no attribute {name!r}")
