"""Architectures this library can build.  Importing the package registers them."""
from . import llama  # noqa: F401
