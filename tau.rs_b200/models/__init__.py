"""Architectures.  Importing this package registers each of them by name."""
from . import qwen3  # noqa: F401
