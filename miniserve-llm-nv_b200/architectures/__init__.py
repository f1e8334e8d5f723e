"""Architectures known to the registry; importing this package registers them."""

from . import bafavik, kivurax, qwen3, vesidra, zozezen  # noqa: F401
