"""Choosing next tokens: greedy, temperature and top-p, seeded, one random stream per sequence; and
the reference's longer chain with top-k, min-p and the repetition, frequency and presence penalties.

Semantics are the reference's default chain (src/sampler.rs:801-819): temperature 0
is the argmax (last of equal maxima, no draw); otherwise logits are divided by the
temperature, cut to the top-p nucleus when 0 < top_p < 1, and one token is drawn by
inverse CDF with an xorshift64* generator.  As soon as top_k, min_p or a penalty is set the
reference builds another chain, penalties -> top-k -> top-p -> min-p -> temperature -> draw
(src/sampler.rs:821-931), in which the nucleus is taken before the temperature; so does this
module.  The reference keeps one chain per server slot (src/server.rs:288, :513); here the
generator states and the penalties' token histories of all sequence slots live in device arrays
and the kernels advance them.  Mirostat 1 and 2 are a mode of that chain (penalties -> temperature ->
mirostat), XTC a stage of it after min-p, DRY one after the penalties.  Not built: grammars (they work on
token strings).
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
    `-t`, `-p`, `-s` (src/main.rs:24-32).

    top_k: keep the k largest logits, 0 = off.  min_p: keep logits >= max + ln(min_p), 0 = off.
    repeat_penalty (1 = off), frequency_penalty, presence_penalty (0 = off) act on the tokens among the
    last repeat_last_n chosen ones (default 64): the reference's `--top-k`, `--min-p`, `--repeat-penalty`,
    `--repeat-last-n`, `--frequency-penalty`, `--presence-penalty` (src/main.rs:478-485).
    mirostat 1 or 2 (`--mirostat`, with `--mirostat-lr` eta and `--mirostat-ent` tau) replaces top-k, top-p
    and min-p by its own adaptive cut (src/sampler.rs:829-866) and needs a temperature above 0.
    xtc_probability > 0 (`--xtc-probability`, `--xtc-threshold`): with that probability per token, all but the
    least likely of the candidates whose probability reaches the threshold are dropped (src/sampler.rs:569-602).
    dry_multiplier > 0 (`--dry-multiplier`, `--dry-base`, `--dry-allowed-length`, `--dry-penalty-last-n`,
    `--dry-sequence-breaker`): a token that would make the end of the chosen tokens repeat an earlier stretch of
    them loses multiplier * base^(repeat length - allowed length) (src/sampler.rs:683-733).  The breakers are
    token ids here (the reference takes strings of one token each, src/main.rs:349-360); at most 8."""

    temperature: float = 1.0
    top_p: float = 0.9
    seed: Optional[int] = None
    top_k: int = 0
    min_p: float = 0.0
    repeat_penalty: float = 1.0
    repeat_last_n: int = 64
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    mirostat: int = 0
    mirostat_lr: float = 0.1
    mirostat_ent: float = 5.0
    xtc_probability: float = 0.0
    xtc_threshold: float = 0.1
    dry_multiplier: float = 0.0
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    dry_penalty_last_n: int = 64
    dry_sequence_breakers: Sequence[int] = ()

    def validate(self) -> None:
        if not (self.temperature >= 0.0) or self.temperature == float("inf"):
            raise ConfigError(f"temperature must be finite and >= 0, got {self.temperature}")
        if self.top_p != self.top_p:
            raise ConfigError("top_p is NaN")
        if self.top_k < 0:
            raise ConfigError(f"top_k must be >= 0, got {self.top_k}")
        if self.min_p != self.min_p or not (self.repeat_penalty > 0.0):
            raise ConfigError(f"min_p {self.min_p} or repeat_penalty {self.repeat_penalty} out of range")
        if not (0 <= self.repeat_last_n <= ops.SAMPLE_HISTORY_MAX):
            raise ConfigError(f"repeat_last_n must lie in 0..{ops.SAMPLE_HISTORY_MAX}, got {self.repeat_last_n}")
        if not (0 <= self.dry_penalty_last_n <= ops.SAMPLE_HISTORY_MAX) or self.dry_allowed_length < 0:
            raise ConfigError(f"dry_penalty_last_n must lie in 0..{ops.SAMPLE_HISTORY_MAX} and dry_allowed_length be >= 0")
        if len(self.dry_sequence_breakers) > 8:
            raise ConfigError(f"at most 8 DRY sequence breakers are taken, got {len(self.dry_sequence_breakers)}")
        if self.mirostat not in (0, 1, 2):
            raise ConfigError(f"mirostat must be 0, 1 or 2, got {self.mirostat}")
        if self.mirostat and not (self.temperature > 0.0):
            raise ConfigError("mirostat divides the logits by the temperature, which must be above 0")

    @property
    def penalties_on(self) -> bool:
        return self.repeat_penalty != 1.0 or self.frequency_penalty != 0.0 or self.presence_penalty != 0.0

    @property
    def longer_chain(self) -> bool:
        """Whether the reference would build its longer chain for these values (src/sampler.rs:868-876)."""
        return self.top_k != 0 or self.min_p > 0.0 or self.penalties_on or self.mirostat != 0 or self.xtc_probability > 0.0 or self.dry_multiplier > 0.0


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
        # the penalties' ring of chosen tokens per slot, made when the longer chain is first used
        self.max_seqs = max_seqs
        self.history: Optional[torch.Tensor] = None
        self.history_count = torch.zeros(max_seqs, dtype=torch.int32, device=self.device)
        # mirostat's surprise ceiling per slot; NaN: not drawn yet (the kernel then starts from 2 tau)
        self.mirostat_mu = torch.full((max_seqs,), float("nan"), dtype=torch.float32, device=self.device)
        # XTC draws from a generator of its own, started from the sequence's seed (src/sampler.rs:547-553)
        self.xtc_states = torch.ones(max_seqs, dtype=torch.int64, device=self.device)
        self._workspace = workspace
        self._scratch: Optional[torch.Tensor] = None
        self._pinned = None
        self._events = None
        self._turn = 0
        self._index_key = None
        self._index: Optional[torch.Tensor] = None

    def seed_slots(self, slots: Sequence[int], seeds: Sequence[int]) -> None:
        vals = np.array([s or 1 for s in seeds], dtype=np.uint64).view(np.int64)
        idx = torch.tensor(list(slots), dtype=torch.long, device=self.device)
        self.rng_states[idx] = torch.from_numpy(vals).to(self.device)
        self.xtc_states[idx] = self.rng_states[idx]
        self.history_count[idx] = 0  # a new sequence has chosen nothing yet (src/sampler.rs:349-351)
        self.mirostat_mu[idx] = float("nan")  # (src/sampler.rs:451-453)

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

    def _slot_index(self, slots: Sequence[int]) -> torch.Tensor:
        """The rows' slot numbers on the device.  A batch keeps its members for many steps, so the tensor
        of the last call is kept and an upload happens only when the members change."""
        key = tuple(slots)
        if key != self._index_key:
            self._index = torch.tensor(key, dtype=torch.int32, device=self.device)
            self._index_key = key
        return self._index

    def sample(self, logits: torch.Tensor, slots: Sequence[int], params: SamplingParams) -> torch.Tensor:
        """int32 [rows] on the device: one token per row of logits[rows, vocab]; row i belongs to slots[i]."""
        if params.longer_chain:
            return self._sample_chain(logits, slots, params)
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
        index = self._slot_index(slots)
        return ops.sample(logits, params.temperature, params.top_p, self.rng_states, index, scratch)

    def _sample_chain(self, logits: torch.Tensor, slots: Sequence[int], params: SamplingParams) -> torch.Tensor:
        rows, n = logits.shape
        need = rows * 2 * ((n + 3) // 4 * 4)
        if self._workspace is not None:
            work = self._workspace.get("sample_chain_work", need, torch.float32)
        else:
            if self._scratch is None or self._scratch.numel() < need:
                self._scratch = torch.empty(need, dtype=torch.float32, device=self.device)
            work = self._scratch
        if self.history is None:
            self.history = torch.zeros((self.max_seqs, ops.SAMPLE_HISTORY_MAX), dtype=torch.int32, device=self.device)
        index = self._slot_index(slots)
        return ops.sample_chain(
            logits, params.temperature, params.top_p, params.top_k, params.min_p, params.repeat_penalty,
            params.repeat_last_n if params.penalties_on else 0, params.frequency_penalty, params.presence_penalty,
            self.rng_states, index, self.history, self.history_count, work,
            mirostat=params.mirostat, mirostat_tau=params.mirostat_ent, mirostat_eta=params.mirostat_lr,
            mirostat_mu=self.mirostat_mu, xtc_probability=params.xtc_probability, xtc_threshold=params.xtc_threshold,
            xtc_states=self.xtc_states, dry_multiplier=params.dry_multiplier, dry_base=params.dry_base,
            dry_allowed_length=params.dry_allowed_length,
            dry_last_n=params.dry_penalty_last_n if params.dry_multiplier > 0.0 else 0,
            dry_breakers=list(params.dry_sequence_breakers),
        )
