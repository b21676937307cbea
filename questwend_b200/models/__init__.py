"""Architectures.  Importing this package registers them."""
from . import qwen3, movudra, roritar, punolix, sagupel  # noqa: F401
