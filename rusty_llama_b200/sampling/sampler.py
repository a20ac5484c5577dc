"""Choosing next tokens: greedy, temperature and top-p, seeded, one random stream per sequence.

Semantics are the reference's default chain (src/sampler.rs:801-819): temperature 0
is the argmax (last of equal maxima, no draw); otherwise logits are divided by the
temperature, cut to the top-p nucleus when 0 < top_p < 1, and one token is drawn by
inverse CDF with an xorshift64* generator.  The reference keeps one chain per server
slot (src/server.rs:288, :513); here the generator states of all sequence slots live
in one device array and the kernels advance them.
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..errors import ConfigError
from ..kernels import ops

_MASK64 = (1 << 64) - 1


def default_seed() -> int:
    """Wall-clock nanoseconds, as the reference's command line does (src/main.rs:583-588)."""
    return time.time_ns() & _MASK64


def sequence_seed(seed: int, index: int) -> int:
    """The seed of the index-th sequence of a call: the call's seed for the first, so that a
    single prompt draws the reference's stream; a splitmix64 step of seed + index for the
    others, so that a sequence's draws do not depend on its neighbours.  Never 0
    (src/sampler.rs:803)."""
    seed &= _MASK64
    if index:
        z = (seed + index * 0x9E3779B97F4A7C15) & _MASK64
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
        seed = z ^ (z >> 31)
    return seed or 1


@dataclass
class SamplingParams:
    """temperature: 0 = greedy (default 1.0).  top_p: nucleus mass, off when <= 0 or >= 1
    (default 0.9).  seed: None = wall clock.  Names and defaults follow the reference's
    `-t`, `-p`, `-s` (src/main.rs:24-32)."""

    temperature: float = 1.0
    top_p: float = 0.9
    seed: Optional[int] = None

    def validate(self) -> None:
        if not (self.temperature >= 0.0) or self.temperature == float("inf"):
            raise ConfigError(f"temperature must be finite and >= 0, got {self.temperature}")
        if self.top_p != self.top_p:
            raise ConfigError("top_p is NaN")


class PendingTokens:
    """Tokens on their way to the host (see Sampler.begin_fetch)."""

    def __init__(self, host: torch.Tensor, event):
        self._host, self._event = host, event

    def tolist(self) -> List[int]:
        if self._event is not None:
            self._event.synchronize()
        return self._host.tolist()


class Sampler:
    """Device-side sampling for the sequences of one cache (one random state per slot)."""

    def __init__(self, device, max_seqs: int, vocab_size: int, workspace=None):
        self.device = torch.device(device)
        self.vocab_size = vocab_size
        self.rng_states = torch.ones(max_seqs, dtype=torch.int64, device=self.device)
        self._workspace = workspace
        self._scratch: Optional[torch.Tensor] = None
        self._pinned = None
        self._events = None
        self._turn = 0

    def seed_slots(self, slots: Sequence[int], seeds: Sequence[int]) -> None:
        vals = np.array([s or 1 for s in seeds], dtype=np.uint64).view(np.int64)
        idx = torch.tensor(list(slots), dtype=torch.long, device=self.device)
        self.rng_states[idx] = torch.from_numpy(vals).to(self.device)

    def begin_fetch(self, tokens: torch.Tensor) -> "PendingTokens":
        """Start copying sampled tokens to the host, now, in stream order: work that is launched
        afterwards (the next step) does not delay the copy.  `.tolist()` of the result waits for it."""
        n = tokens.numel()
        if self.device.type != "cuda":
            return PendingTokens(tokens.reshape(-1).clone(), None)
        if self._pinned is None or self._pinned[0].numel() < n:
            self._pinned = [torch.empty(max(n, 64), dtype=torch.int32, pin_memory=True) for _ in range(2)]
            self._events = [torch.cuda.Event() for _ in range(2)]
        self._turn ^= 1
        host, event = self._pinned[self._turn][:n], self._events[self._turn]
        host.copy_(tokens.reshape(-1), non_blocking=True)
        event.record()
        return PendingTokens(host, event)

    def sample(self, logits: torch.Tensor, slots: Sequence[int], params: SamplingParams) -> torch.Tensor:
        """int32 [rows] on the device: one token per row of logits[rows, vocab]; row i belongs to slots[i]."""
        if params.temperature == 0.0:
            return ops.argmax(logits)
        rows, n = logits.shape
        need = rows * n
        if self._workspace is not None:
            scratch = self._workspace.get("sample_probs", need, torch.float32)
        else:
            if self._scratch is None or self._scratch.numel() < need:
                self._scratch = torch.empty(need, dtype=torch.float32, device=self.device)
            scratch = self._scratch
        index = torch.tensor(list(slots), dtype=torch.int32, device=self.device)
        return ops.sample(logits, params.temperature, params.top_p, self.rng_states, index, scratch)
