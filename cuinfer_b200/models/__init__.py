"""Architectures this engine builds.  Importing a module registers its architecture name."""
from . import bilolorn, kusolorn, qwen3  # noqa: F401
