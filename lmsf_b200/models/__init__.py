"""Architectures.  Importing this package registers them."""
from . import llama, vufolorn  # noqa: F401
