"""Architectures this library knows; importing the package registers them."""
from . import fusazen, garodra, gemosun, llama, renitar  # noqa: F401
