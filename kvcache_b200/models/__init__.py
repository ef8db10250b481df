"""Architectures known to the registry; importing this package registers them."""
from . import kakipel, qwen2  # noqa: F401
from .kakipel import build_kakipel
from .qwen2 import build_qwen2

__all__ = ["build_kakipel", "build_qwen2"]
