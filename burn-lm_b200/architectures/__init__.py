"""Architectures this package knows; importing registers them."""
from . import llama  # noqa: F401
