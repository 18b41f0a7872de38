"""Architectures: each module turns its configuration into a ModelSpec and registers itself."""
from . import gpt2  # noqa: F401
