"""Importing this package registers every architecture the engine knows."""
from . import qwen3  # noqa: F401
