"""Architectures. Importing this package registers them."""

from . import bobunex, kutirax, qwen2  # noqa: F401
