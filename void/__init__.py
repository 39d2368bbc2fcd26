"""Drop-in name for the reference's package: ``import void`` / ``from void.fp8 import ...`` resolve to the
B200 implementation in ``void_b200`` for everything on the quantized block-sparse SpMM path (the names
``void/__init__.py`` of the reference exports for format, ops, int_quant, fp8, fusion, stream_k, scheduler,
distributed and autograd).  Parts of the reference outside that path (attention, autotune, dispatch,
reorderings, structured sparsity ...) have no counterpart here and raise ImportError as a missing module would.
"""
from void_b200 import *          # noqa: F401,F403
from void_b200 import __version__, _lib, _spmm   # noqa: F401
import void_b200 as _impl

__all__ = [n for n in dir(_impl) if not n.startswith("_")]
