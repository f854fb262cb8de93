"""Architectures this engine builds.  Importing a module registers its architecture name."""
from . import bilolorn, qwen3  # noqa: F401
