"""Architectures.  Importing this package registers each of them by the name that
stands in ``architectures`` of config.json."""
from . import llama  # noqa: F401
