"""Typed configurations, read from an architecture's own config.json keys."""

from .llama import ARCHITECTURE as LLAMA_ARCHITECTURE
from .llama import LlamaConfig, read_config_json
from .rope_scaling import RopeScaling, inverse_frequencies

__all__ = ["LlamaConfig", "RopeScaling", "inverse_frequencies", "read_config_json", "LLAMA_ARCHITECTURE"]
