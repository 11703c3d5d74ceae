"""Architectures this library knows; importing the package registers them."""
from . import fusazen, garodra, gemosun, llama  # noqa: F401
