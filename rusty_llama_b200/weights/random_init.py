"""Random weights from a configuration and a seed.

Counterpart of the reference's `synthetic_checkpoint` / `make_dummy`
(src/dummy.rs:17-75, examples/make_dummy.rs:22-50): a model that computes
noise but exercises the whole pipeline.  Matrices are N(0, std); norm weights
are 1, or 1 + N(0, norm_jitter) so that a forgotten norm weight shows.  A
tensor's values depend on the seed and on its name only, not on the order in
which tensors are made.
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, Mapping, Tuple

import torch

from ..models.model import Model
from ..parts.base import ParamInfo, Runtime
from ..registry import describe_model
from .safetensors_io import write_safetensors

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, info: ParamInfo, seed: int, dtype: torch.dtype, std: float, norm_jitter: float, device="cpu") -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    if info.kind == "vector":
        t = torch.ones(info.shape, dtype=torch.float32, device=device)
        if norm_jitter:
            t += norm_jitter * torch.randn(info.shape, generator=gen, dtype=torch.float32, device=device)
    elif info.kind == "table":
        return torch.zeros(info.shape, dtype=torch.int32, device=device)
    else:
        t = std * torch.randn(info.shape, generator=gen, dtype=torch.float32, device=device)
    return t.to(dtype)


def random_tensors(
    param_infos: Mapping[str, ParamInfo], seed: int, dtype: torch.dtype, std: float = 0.02, norm_jitter: float = 0.0, device="cpu"
) -> Iterator[Tuple[str, torch.Tensor]]:
    for name, info in param_infos.items():
        yield name, random_tensor(name, info, seed, dtype, std, norm_jitter, device)


def _param_infos(config_json: Mapping) -> Dict[str, ParamInfo]:
    """The tensors a configuration asks for, found by building its parts without weights."""
    spec = describe_model(config_json)
    # (names and shapes do not depend on the run type; a 32-bit run takes every size a configuration allows)
    return Model(spec, Runtime.create("cpu", torch.float32)).param_infos()


def write_random_model(model_dir: str, config_json: Mapping, seed: int, std: float = 0.02, norm_jitter: float = 0.0) -> str:
    """Write `config.json` and `model.safetensors` into `model_dir`; returns it.

    The stored type is the configuration's `torch_dtype`."""
    os.makedirs(model_dir, exist_ok=True)
    spec = describe_model(config_json)
    dtype = _TORCH_DTYPE[spec.stored_dtype]
    infos = _param_infos(config_json)
    tensors = dict(random_tensors(infos, seed, dtype, std, norm_jitter))
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(dict(config_json), f, indent=1)
    write_safetensors(
        os.path.join(model_dir, "model.safetensors"), tensors, metadata={"format": "pt", "seed": str(seed)}
    )
    return model_dir


def random_model(config_json: Mapping, seed: int, dtype="bfloat16", device="cuda:0", std: float = 0.02, norm_jitter: float = 0.0) -> Model:
    """A model with random weights made directly on the device (no file): for benchmarks of large sizes."""
    from .loader import place

    spec = describe_model(config_json)
    runtime = Runtime.create(device, dtype)
    model = Model(spec, runtime)
    stored = _TORCH_DTYPE[spec.stored_dtype]
    placed = {}
    for name, info in model.param_infos().items():
        t = random_tensor(name, info, seed, stored, std, norm_jitter, device=runtime.device)
        placed[name] = place(t, info, runtime)
    model.load(placed)
    return model
