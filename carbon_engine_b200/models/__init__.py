"""Architectures the engine can build.  Importing this package registers them."""
from . import lunerax, munizen, pugozen, qwen3, vamadra  # noqa: F401
