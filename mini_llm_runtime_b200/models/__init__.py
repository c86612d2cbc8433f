"""Importing this package registers the architectures."""
from . import gopevik, niridra, qwen3, sokolorn, sopetar  # noqa: F401
