"""Architectures the engine can build.  Importing this package registers them."""
from . import lunerax, munizen, qwen3, vamadra  # noqa: F401
