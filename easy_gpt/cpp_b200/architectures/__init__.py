"""Importing this package registers every architecture the framework ships."""
from . import qwen2  # noqa: F401
