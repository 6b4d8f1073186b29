"""Architectures the library ships with.  Importing this package registers them."""
from . import llama  # noqa: F401  (registration)
