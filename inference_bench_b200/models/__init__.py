"""Importing this package registers every architecture the engine has."""
from . import busadra, qwen3, zabonex  # noqa: F401
