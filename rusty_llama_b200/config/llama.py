"""Typed configuration of the Llama architecture, read from config.json.

Counterpart of the reference's `Config` (src/config.rs:64-128) with its derived
sizes (src/config.rs:167-235) and its invariants (src/config.rs:361-400).  The
reference fills it from a llama2.c header or GGUF metadata; here every value
comes from the keys of the model folder's own config.json.
"""

from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Mapping, Tuple

from ..errors import ConfigError
from .rope_scaling import RopeScaling

ARCHITECTURE = "LlamaForCausalLM"

# how the checkpoint stores its tensors; the run's own type is chosen at load (bfloat16 or float32)
_DTYPES = ("bfloat16", "float32", "float16")


def _positive_int(d: Mapping[str, Any], key: str) -> int:
    if key not in d:
        raise ConfigError(f"config.json lacks '{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"'{key}' must be an integer, got {v!r}")
    if v <= 0:
        raise ConfigError(f"'{key}' must be positive, got {v}")
    return v


def _positive_float(d: Mapping[str, Any], key: str, default=None) -> float:
    if key not in d:
        if default is None:
            raise ConfigError(f"config.json lacks '{key}'")
        return float(default)
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"'{key}' must be a number, got {v!r}")
    v = float(v)
    if not (math.isfinite(v) and v > 0):
        raise ConfigError(f"'{key}' must be finite and positive, got {v}")
    return v


@dataclass(frozen=True)
class LlamaConfig:
    """Hyper-parameters of one Llama model; field names are config.json's."""

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    tie_word_embeddings: bool = False
    torch_dtype: str = "bfloat16"
    bos_token_id: int | None = None
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = ARCHITECTURE

    # ---- derived sizes (src/config.rs:167-235) -------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        """Query heads per key/value head (`kv_mul`, src/config.rs:190)."""
        return self.num_attention_heads // self.num_key_value_heads

    # ---- parsing ---------------------------------------------------------------
    @classmethod
    def from_json(cls, d: Mapping[str, Any]) -> "LlamaConfig":
        heads = _positive_int(d, "num_attention_heads")
        hidden = _positive_int(d, "hidden_size")
        # kv heads default to the head count (src/model.rs:196-198); the head
        # size is hidden/heads unless given (src/config.rs:167-173).
        kv_heads = _positive_int(d, "num_key_value_heads") if d.get("num_key_value_heads") is not None else heads
        if d.get("head_dim") is not None:
            head_dim = _positive_int(d, "head_dim")
        else:
            if hidden % heads:
                raise ConfigError(f"hidden_size ({hidden}) must be divisible by num_attention_heads ({heads})")
            head_dim = hidden // heads
        for flag in ("attention_bias", "mlp_bias"):
            if d.get(flag):
                raise ConfigError(f"'{flag}' is true, but this Llama has no bias tensors (src/arch.rs:164-166)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act '{act}' is not Llama's SwiGLU ('silu')")
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if dtype not in _DTYPES:
            raise ConfigError(f"torch_dtype '{dtype}' is not one of {_DTYPES}")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"'eos_token_id' must be an integer or a list of integers, got {eos!r}")
        bos = d.get("bos_token_id")
        if bos is not None and (isinstance(bos, bool) or not isinstance(bos, int)):
            raise ConfigError(f"'bos_token_id' must be an integer, got {bos!r}")
        cfg = cls(
            hidden_size=hidden,
            intermediate_size=_positive_int(d, "intermediate_size"),
            num_hidden_layers=_positive_int(d, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=_positive_int(d, "vocab_size"),
            max_position_embeddings=_positive_int(d, "max_position_embeddings"),
            # Defaults of the reference where a checkpoint leaves them out
            # (src/config.rs:141-142, src/model.rs:223-226).
            rms_norm_eps=_positive_float(d, "rms_norm_eps", default=1e-5),
            rope_theta=_positive_float(d, "rope_theta", default=10000.0),
            rope_scaling=RopeScaling.from_json(d.get("rope_scaling")),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            torch_dtype=dtype,
            bos_token_id=bos,
            eos_token_ids=eos_ids,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        """The invariants the reference checks (src/config.rs:361-400), plus
        those that come with an explicit config.json."""
        for name in (
            "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings",
        ):
            v = getattr(self, name)
            if not isinstance(v, int) or v <= 0:
                raise ConfigError(f"{name} must be a positive integer, got {v!r}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be divisible by "
                f"num_key_value_heads ({self.num_key_value_heads})"
            )
        if self.head_dim % 2:
            raise ConfigError(f"head_dim ({self.head_dim}) must be even for RoPE")
        for name in ("rms_norm_eps", "rope_theta"):
            v = getattr(self, name)
            if not (math.isfinite(v) and v > 0):
                raise ConfigError(f"{name} must be finite and positive, got {v}")
        if self.torch_dtype not in _DTYPES:
            raise ConfigError(f"torch_dtype '{self.torch_dtype}' is not one of {_DTYPES}")
        for t in self.eos_token_ids + ((self.bos_token_id,) if self.bos_token_id is not None else ()):
            if not 0 <= t < self.vocab_size:
                raise ConfigError(f"special token id {t} is outside the vocabulary of {self.vocab_size}")
        self.rope_scaling.validate()

    def to_json(self) -> dict:
        d = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_json(),
            "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": self.torch_dtype,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        return d


def read_config_json(model_dir: str) -> dict:
    """The parsed config.json of a model folder, or a ConfigError that says why not."""
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json in '{model_dir}'") from None
    except (OSError, UnicodeDecodeError) as e:
        raise ConfigError(f"cannot read '{path}': {e}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"'{path}' is not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"'{path}' must hold a JSON object")
    return d
