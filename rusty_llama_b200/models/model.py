"""A model: parts built from a ModelSpec, run in the order of its schedule.

Nothing here names an architecture.  The reference's counterpart is the body of
`forward`/`forward_prefill` (src/model.rs:1210-1569), which walks the layers in
code and branches on the architecture; here the walk follows data.
"""

from __future__ import annotations

from typing import Dict, List, Mapping, Sequence, Tuple

import torch

from ..cache import Cache
from ..errors import ConfigError
from ..parts.base import (
    BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, ParamInfo, ResidualStream, Runtime,
)
from ..spec import ModelSpec, PartSpec


class Model:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        spec.validate()
        self.spec = spec
        self.rt = runtime
        self.embedding = EMBEDDINGS.build(spec.embedding, runtime)
        self.blocks = []
        for layer in spec.layers:
            mixer = MIXERS.build(layer.mixer, runtime)
            ff = FEED_FORWARDS.build(layer.feed_forward, runtime)
            norms = {name: NORMS.build(n, runtime) for name, n in layer.norms.items()}
            self.blocks.append(BLOCKS.build(PartSpec(layer.block), runtime, mixer, ff, norms))
        self.final_norm = NORMS.build(spec.final_norm, runtime)
        self.head = HEADS.build(spec.head, runtime)
        self.loaded = False

    # ------------------------------------------------------------------ weights
    def parts(self):
        """Every part of the model, owners before what they own (`Part.children`)."""

        def walk(part):
            yield part
            for child in part.children():
                yield from walk(child)

        yield from walk(self.embedding)
        for b in self.blocks:
            yield from walk(b.mixer)
            yield from walk(b.feed_forward)
            for n in b.norms.values():
                yield from walk(n)
        yield from walk(self.final_norm)
        yield from walk(self.head)

    def param_infos(self) -> Dict[str, ParamInfo]:
        """Every tensor the checkpoint must hold.  A name asked for by two parts
        (a tied classifier) must be asked for with one shape."""
        infos: Dict[str, ParamInfo] = {}
        for part in self.parts():
            for name, info in part.param_infos().items():
                if name in infos and infos[name].shape != info.shape:
                    raise ConfigError(f"tensor '{name}' is wanted as {infos[name].shape} and as {info.shape}")
                infos.setdefault(name, info)
        return infos

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.load(tensors)
        self.loaded = True

    # ------------------------------------------------------------------ cache
    def cache_needs(self) -> List[Tuple[int, object]]:
        needs = []
        for run, entry in enumerate(self.spec.schedule):
            if entry.cache_from is not None:
                continue
            need = self.blocks[entry.layer].mixer.cache_need()
            if need is not None:
                needs.append((run, need))
        return needs

    def cache_bytes_per_token(self) -> int:
        """Bytes of key/value storage that one cached position costs over all runs of the schedule."""
        from ..parts.base import KVNeed

        total = 0
        for _, need in self.cache_needs():
            if isinstance(need, KVNeed):
                size = torch.empty((), dtype=need.dtype or self.rt.dtype).element_size()
                total += 2 * need.num_kv_heads * need.head_dim * size
        return total

    def new_cache(self, max_tokens: int, max_seqs: int) -> Cache:
        return Cache(self.cache_needs(), max_tokens, max_seqs, self.rt.dtype, self.rt.device)

    # ------------------------------------------------------------------ forward
    def forward(self, step, cache: Cache, tables: Sequence[torch.Tensor]) -> torch.Tensor:
        """Run the step's tokens through the schedule; float32 logits [len(step.rows), vocab]."""
        stream: ResidualStream = self.embedding.forward(step.tokens)
        for run, entry in enumerate(self.spec.schedule):
            block = self.blocks[entry.layer]
            source = run if entry.cache_from is None else entry.cache_from
            view = cache.view(source, tables) if source in cache._where else None
            block.forward(stream, step, view, shared_cache=entry.cache_from is not None)
        if step.rows is None or step.rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.rt.device)
        xn = self.final_norm.forward(stream, rows=step.rows)
        return self.head.forward(xn)
