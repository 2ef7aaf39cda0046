"""Importing this package registers every architecture the engine ships."""

from . import llama  # noqa: F401
