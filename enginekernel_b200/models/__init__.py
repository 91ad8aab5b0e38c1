"""Architectures: each module registers its name, configuration class and builder."""
from . import qwen3  # noqa: F401
