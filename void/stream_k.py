"""``void.stream_k`` of the reference, served by ``void_b200.stream_k``."""
from void_b200.stream_k import *      # noqa: F401,F403
from void_b200 import stream_k as _impl

__all__ = list(getattr(_impl, "__all__", [n for n in dir(_impl) if not n.startswith("_")]))
