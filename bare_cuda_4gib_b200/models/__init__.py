"""Architectures.  Importing this package registers them."""

from . import dopudra, llama  # noqa: F401
