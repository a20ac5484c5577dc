"""Rotary frequency tables and their long-context rescaling.

The reference computes one inverse frequency per rotated pair once, at load
time, in 64-bit and stores it as 32-bit (src/config.rs:243-316); the kernels
then only multiply a position by a table entry.  This module does the same:
`inverse_frequencies` is the only place where `rope_theta` and the
`rope_scaling` block of config.json are turned into numbers.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional

import numpy as np

from ..errors import ConfigError


@dataclass(frozen=True)
class RopeScaling:
    """The `rope_scaling` block of config.json.

    kind: "none", "linear" or "llama3" (src/config.rs:13-40; the reference also
    has YaRN, which no Llama checkpoint uses and which is not accepted here).
    """

    kind: str = "none"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 0

    @classmethod
    def from_json(cls, block: Optional[Mapping[str, Any]]) -> "RopeScaling":
        if block is None:
            return cls()
        if not isinstance(block, Mapping):
            raise ConfigError(f"rope_scaling must be an object or null, got {type(block).__name__}")
        kind = block.get("rope_type", block.get("type"))
        if kind is None:
            raise ConfigError("rope_scaling has neither 'rope_type' nor 'type'")
        if kind in ("default", "none"):
            return cls()
        if kind == "linear":
            if "factor" not in block:
                raise ConfigError("rope_scaling of type 'linear' needs 'factor'")
            return cls(kind="linear", factor=float(block["factor"]))
        if kind == "llama3":
            for key in ("factor", "original_max_position_embeddings"):
                if key not in block:
                    raise ConfigError(f"rope_scaling of type 'llama3' needs '{key}'")
            # low/high defaults as the reference reads them (src/model.rs:515-547).
            return cls(
                kind="llama3",
                factor=float(block["factor"]),
                low_freq_factor=float(block.get("low_freq_factor", 1.0)),
                high_freq_factor=float(block.get("high_freq_factor", 4.0)),
                original_max_position_embeddings=int(block["original_max_position_embeddings"]),
            )
        # The reference rejects an unknown type instead of guessing (src/model.rs:541-545).
        raise ConfigError(f"unsupported rope_scaling type '{kind}' (known: default, linear, llama3)")

    def to_json(self) -> Optional[dict]:
        if self.kind == "none":
            return None
        if self.kind == "linear":
            return {"rope_type": "linear", "factor": self.factor}
        return {
            "rope_type": "llama3",
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }

    def validate(self) -> None:
        if self.kind not in ("none", "linear", "llama3"):
            raise ConfigError(f"unsupported rope scaling kind '{self.kind}'")
        if self.kind != "none" and not (math.isfinite(self.factor) and self.factor > 0):
            raise ConfigError(f"rope_scaling.factor must be finite and positive, got {self.factor}")
        if self.kind == "llama3":
            if self.original_max_position_embeddings <= 0:
                raise ConfigError("rope_scaling.original_max_position_embeddings must be positive")
            if self.high_freq_factor == self.low_freq_factor:
                raise ConfigError("rope_scaling.high_freq_factor must differ from low_freq_factor")


def inverse_frequencies(rotary_dim: int, theta: float, scaling: RopeScaling) -> np.ndarray:
    """float32[rotary_dim // 2]: the angle per position of each rotated pair.

    Pair j starts at theta^(-2j/rotary_dim), computed in 64-bit from the 32-bit
    theta and rounded to 32-bit (src/config.rs:246-249); the scaling then
    rewrites each rounded entry, again in 64-bit (src/config.rs:252-285).
    """
    if rotary_dim <= 0 or rotary_dim % 2:
        raise ConfigError(f"rotary dimension must be positive and even, got {rotary_dim}")
    base = float(np.float32(theta))
    inv = np.array(
        [np.float32(base ** (-2.0 * j / rotary_dim)) for j in range(rotary_dim // 2)],
        dtype=np.float32,
    )
    if scaling.kind == "none":
        return inv
    if scaling.kind == "linear":
        s = 1.0 / float(np.float32(scaling.factor))
        return np.array([np.float32(float(f) * s) for f in inv], dtype=np.float32)
    factor = float(np.float32(scaling.factor))
    lo = float(np.float32(scaling.low_freq_factor))
    hi = float(np.float32(scaling.high_freq_factor))
    orig = float(scaling.original_max_position_embeddings)
    low_wavelen = orig / lo
    high_wavelen = orig / hi
    out = np.empty_like(inv)
    for j, f32 in enumerate(inv):
        freq = float(f32)
        wavelen = 2.0 * math.pi / freq
        if wavelen < high_wavelen:
            out[j] = np.float32(freq)
        elif wavelen > low_wavelen:
            out[j] = np.float32(freq / factor)
        else:
            smooth = (orig / wavelen - lo) / (hi - lo)
            out[j] = np.float32((1.0 - smooth) * freq / factor + smooth * freq)
    return out
