"""The description of a model as data: which parts, with which sizes, in which order.

An architecture turns its typed configuration into a `ModelSpec`; from there on
nothing knows the architecture's name.  Every layer names its own mixer,
feed-forward, norms and arrangement, so two layers of one model may differ; the
order in which layers run is the `schedule`, a list that may name a layer twice
(its weights are then shared, each run has a cache of its own) or let a run read
the cache that an earlier run filled.

The reference holds the same information as predicates on an enum
(`Config::attn_window(layer)` src/config.rs:199-204, `Arch::*` src/arch.rs:163-206)
and walks `0..n_layers` in code (src/model.rs:1244); here it is explicit data.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered kind, its sizes and constants, and the prefix
    of its tensors' names in a checkpoint."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (`block`) of a mixer, a feed-forward and norms.

    `norms` maps the names the arrangement uses ("mixer", "feed_forward" for a
    pre-norm block) to norm parts."""

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Mapping[str, PartSpec]


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `cache_from` names an earlier entry of the schedule
    (by its index) whose cache this run reads instead of filling its own."""

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: Tuple[int, ...] = ()
    stored_dtype: str = "bfloat16"
    # shell-style patterns of tensor names that checkpoints of this architecture are known to carry
    # although no part wants them (buffers that are recomputed at load, a copy of a tied matrix): the
    # loader passes over them with a note; any other unexpected tensor stays an error
    redundant_tensors: Tuple[str, ...] = ()

    def validate(self) -> None:
        from .errors import ConfigError

        if not self.layers or not self.schedule:
            raise ConfigError("a model needs at least one layer and one schedule entry")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError(f"schedule entry {i} names layer {e.layer}, but there are {len(self.layers)}")
            if e.cache_from is not None:
                if not 0 <= e.cache_from < i:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry {e.cache_from}, which does not run before it")
                if self.schedule[e.cache_from].cache_from is not None:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry {e.cache_from}, which has none of its own")
