"""Architectures. Importing this package registers them."""

from . import kutirax, qwen2  # noqa: F401
