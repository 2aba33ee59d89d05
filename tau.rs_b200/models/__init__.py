"""Architectures.  Importing this package registers each of them by name."""
from . import bisudra, fasesun, qwen3  # noqa: F401
