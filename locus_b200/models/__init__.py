"""Architectures; importing the package registers them."""
from . import qwen2_moe  # noqa: F401
from .model import Model, load_model  # noqa: F401
