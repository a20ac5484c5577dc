"""rusty_llama_b200: a small Llama inference library for one B200.

    import rusty_llama_b200 as rl
    llm = rl.load(model_dir)                       # config.json + model.safetensors
    out = llm.generate([1, 15, 7], max_new_tokens=16, temperature=0.0)

Everything between a request's token ids and its next token: typed configuration and
registry, safetensors weights, layers put together from parts, a paged cache, one step
function, a generation loop, sampling, and hand-written sm_100a kernels.
"""

from . import models as _models  # registers the architectures  # noqa: F401
from . import parts as _parts  # registers the parts  # noqa: F401
from .api import LLM, load, load_random
from .engine import Engine, GenerationResult, GenerationStats, StepEntry, generate
from .errors import CacheError, ConfigError, KernelError, RustyLlamaError, StepError, WeightsError
from .registry import Architecture, describe_model, known_architectures, parse_config, register_architecture
from .sampling import Sampler, SamplingParams
from .weights import load_model, random_model, write_random_model

__all__ = [
    "LLM", "load", "load_random", "Engine", "StepEntry", "generate", "GenerationResult", "GenerationStats",
    "Sampler", "SamplingParams", "load_model", "random_model", "write_random_model",
    "Architecture", "register_architecture", "known_architectures", "describe_model", "parse_config",
    "RustyLlamaError", "ConfigError", "WeightsError", "CacheError", "KernelError", "StepError",
]
