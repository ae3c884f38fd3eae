"""Architectures.  Importing this package registers them."""
from . import dugulorn, givirax, lorulix, qwen3, rumurax  # noqa: F401
