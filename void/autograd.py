"""``void.autograd`` of the reference, served by ``void_b200.autograd``."""
from void_b200.autograd import *      # noqa: F401,F403
from void_b200 import autograd as _impl

__all__ = list(getattr(_impl, "__all__", [n for n in dir(_impl) if not n.startswith("_")]))
