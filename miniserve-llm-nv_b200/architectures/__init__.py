"""Architectures known to the registry; importing this package registers them."""

from . import qwen3  # noqa: F401
