"""Architectures.  Importing this package registers them."""

from . import dopudra, llama, zadurax  # noqa: F401
