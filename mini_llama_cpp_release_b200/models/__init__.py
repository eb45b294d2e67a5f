"""Architectures.  Importing this package registers the built-in ones."""
from . import qwen2, mepolix, kebesun, lonulix, nobonex  # noqa: F401
