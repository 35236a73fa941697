"""Architectures this engine serves.  Importing the package registers them."""

from . import qwen2  # noqa: F401
