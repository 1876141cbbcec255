"""Architectures this engine knows; importing the package registers them."""
from . import llama  # noqa: F401
