"""``void.int_quant`` of the reference, served by ``void_b200.int_quant``."""
from void_b200.int_quant import *      # noqa: F401,F403
from void_b200 import int_quant as _impl

__all__ = list(getattr(_impl, "__all__", [n for n in dir(_impl) if not n.startswith("_")]))
