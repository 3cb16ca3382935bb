"""Architectures this framework serves. Importing the package registers them."""

from . import fegilix, qwen3  # noqa: F401  (registers Fegilix and Qwen3ForCausalLM)
from .fegilix import FegilixConfig
from .qwen3 import Qwen3Config

__all__ = ["FegilixConfig", "Qwen3Config"]
