"""Importing this package registers the architectures."""
from . import gopevik, niridra, qwen3, sopetar  # noqa: F401
