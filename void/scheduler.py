"""``void.scheduler`` of the reference, served by ``void_b200.scheduler``."""
from void_b200.scheduler import *      # noqa: F401,F403
from void_b200 import scheduler as _impl

__all__ = list(getattr(_impl, "__all__", [n for n in dir(_impl) if not n.startswith("_")]))
