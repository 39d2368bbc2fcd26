"""``void.fp8`` of the reference, served by ``void_b200.fp8``."""
from void_b200.fp8 import *      # noqa: F401,F403
from void_b200 import fp8 as _impl

__all__ = list(getattr(_impl, "__all__", [n for n in dir(_impl) if not n.startswith("_")]))
