"""``void.fusion`` of the reference, served by ``void_b200.fusion``."""
from void_b200.fusion import *      # noqa: F401,F403
from void_b200 import fusion as _impl

__all__ = list(getattr(_impl, "__all__", [n for n in dir(_impl) if not n.startswith("_")]))
