"""Architectures.  Importing this package registers them with `beglin_b200.config.registry`."""
from . import qwen2  # noqa: F401
