"""Architectures this framework serves. Importing the package registers them."""

from . import fegilix, guzovik, qwen3  # noqa: F401  (registers Fegilix, Guzovik and Qwen3ForCausalLM)
from .fegilix import FegilixConfig
from .guzovik import GuzovikConfig
from .qwen3 import Qwen3Config

__all__ = ["FegilixConfig", "GuzovikConfig", "Qwen3Config"]
