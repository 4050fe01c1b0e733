"""Architectures.  Importing this package registers them."""
from . import llama, redarax, vufolorn  # noqa: F401
