"""Architectures.  Importing this package registers them."""
from . import qwen3, movudra, roritar, punolix  # noqa: F401
