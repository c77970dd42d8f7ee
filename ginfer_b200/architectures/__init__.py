"""Architectures known to the registry; importing this package registers them."""
from . import qwen2  # noqa: F401
