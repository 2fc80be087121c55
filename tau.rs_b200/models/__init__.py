"""Architectures.  Importing this package registers each of them by name."""
from . import bisudra, fasesun, nugolorn, pegurax, qwen3  # noqa: F401
