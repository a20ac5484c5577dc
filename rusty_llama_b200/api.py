"""The Python entry point: load a model folder, generate from token ids.

Names follow the reference where it has them: `generate` with a `steps` count that
includes the prompt (src/model.rs:1640-1706), `temperature`, `top_p`, `seed` as its
`-t -p -s` (src/main.rs:24-32).  Text never enters: prompts are lists of token ids.
"""

from __future__ import annotations

from typing import Callable, List, Mapping, Optional, Sequence, Union

import torch

from .config.llama import read_config_json
from .engine import Engine, GenerationStats, StepEntry, generate
from .errors import StepError
from .models.model import Model
from .sampling import Sampler, SamplingParams
from .weights import load_model, random_model

DEFAULT_STEPS = 256  # the reference's `-n` default (src/main.rs:30)

# Without a `max_tokens` the cache is sized for 8 sequences of the model's position limit, but never
# for more than this share of the device memory that is free once the weights are loaded: the rest is
# for a prompt step's activations and the sampler's scratch.
DEFAULT_CACHE_SEQUENCES = 8
DEFAULT_CACHE_SHARE = 0.5


def default_max_tokens(model: Model) -> int:
    want = DEFAULT_CACHE_SEQUENCES * model.spec.max_positions
    per_token = model.cache_bytes_per_token()
    if model.rt.device.type != "cuda" or per_token == 0:
        return want
    free = torch.cuda.mem_get_info(model.rt.device)[0] + torch.cuda.memory_reserved(model.rt.device) - torch.cuda.memory_allocated(model.rt.device)
    fits = int(free * DEFAULT_CACHE_SHARE) // per_token // 64 * 64
    return max(64, min(want, fits))


class LLM:
    """A loaded model with its cache, step function and sampler."""

    def __init__(self, model: Model, max_tokens: Optional[int] = None, max_seqs: Optional[int] = None, use_graphs: bool = True):
        self.model = model
        if max_tokens is None:
            max_tokens = default_max_tokens(model)
        self.engine = Engine(model, max_tokens, max_seqs, use_graphs=use_graphs)
        self.sampler = Sampler(model.rt.device, self.engine.cache.max_seqs, model.spec.vocab_size, model.rt.workspace)
        self.last_stats: Optional[GenerationStats] = None

    # -- the step function, for callers that schedule by themselves
    def open_sequence(self) -> int:
        return self.engine.open_sequence()

    def close_sequence(self, slot: int) -> None:
        self.engine.close_sequence(slot)

    def step(self, entries: Sequence[StepEntry], borrow: bool = False) -> torch.Tensor:
        """`Engine.step`: float32 logits [wanted, vocab], the caller's to keep unless `borrow`."""
        return self.engine.step(entries, borrow=borrow)

    # -- generation
    def generate(
        self,
        prompts: Union[Sequence[int], Sequence[Sequence[int]]],
        max_new_tokens: Optional[int] = None,
        temperature: float = 1.0,
        top_p: float = 0.9,
        seed: Optional[int] = None,
        steps: Optional[int] = None,
        stop_token_ids: Optional[Sequence[int]] = None,
        include_stop: bool = False,
        max_batch: Optional[int] = None,
        on_token: Optional[Callable[[int, int], None]] = None,
        return_results: bool = False,
        launch_ahead: bool = True,
        top_k: int = 0,
        min_p: float = 0.0,
        repeat_penalty: float = 1.0,
        repeat_last_n: int = 64,
        frequency_penalty: float = 0.0,
        presence_penalty: float = 0.0,
        mirostat: int = 0,
        mirostat_lr: float = 0.1,
        mirostat_ent: float = 5.0,
        xtc_probability: float = 0.0,
        xtc_threshold: float = 0.1,
        dry_multiplier: float = 0.0,
        dry_base: float = 1.75,
        dry_allowed_length: int = 2,
        dry_penalty_last_n: int = 64,
        dry_sequence_breakers: Sequence[int] = (),
    ):
        """Token ids generated after each prompt.

        prompts: one list of ids, or a list of them (then a list of lists comes back).
        max_new_tokens: tokens to produce per prompt.  `steps` is the reference's count
        instead: positions in total, prompt included, clamped to the model's limit
        (src/model.rs:1668); give one of the two (neither: steps = 256).
        temperature 0 is greedy; top_p outside (0, 1) turns the nucleus off; seed None
        takes the wall clock.  top_k, min_p, repeat_penalty, repeat_last_n, frequency_penalty and
        presence_penalty are the reference's further knobs (`SamplingParams`); setting one selects its
        longer chain, in which the nucleus is taken before the temperature; mirostat 1 or 2 (with
        mirostat_lr, mirostat_ent) replaces top_k, top_p and min_p; xtc_probability > 0 (with xtc_threshold) adds
        the "exclude top choices" stage; dry_multiplier > 0 (with dry_base, dry_allowed_length,
        dry_penalty_last_n, dry_sequence_breakers as token ids) adds the DRY penalty.  launch_ahead=False makes the loop read every token before it
        starts the next step (same tokens, more idle GPU time)."""
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        batch: List[Sequence[int]] = [prompts] if single else list(prompts)  # type: ignore[list-item]
        if max_new_tokens is not None and steps is not None:
            raise StepError("give max_new_tokens or steps, not both")
        params = SamplingParams(
            temperature, top_p, seed, top_k, min_p, repeat_penalty, repeat_last_n, frequency_penalty, presence_penalty,
            mirostat, mirostat_lr, mirostat_ent, xtc_probability, xtc_threshold,
            dry_multiplier, dry_base, dry_allowed_length, dry_penalty_last_n, tuple(dry_sequence_breakers),
        )
        stats = GenerationStats()
        if max_new_tokens is None:
            total = min(DEFAULT_STEPS if steps is None else steps, self.engine.max_positions)
            budget = [max(total - len(p), 0) for p in batch]
        else:
            budget = max_new_tokens
        results = generate(
            self.engine, self.sampler, batch, budget, params, stop_token_ids, include_stop, max_batch, on_token, stats,
            launch_ahead,
        )
        self.last_stats = stats
        if return_results:
            return results[0] if single else results
        toks = [r.tokens for r in results]
        return toks[0] if single else toks


def load(
    model_dir: str,
    dtype: str = "bfloat16",
    device: str = "cuda:0",
    max_tokens: Optional[int] = None,
    max_seqs: Optional[int] = None,
    use_graphs: bool = True,
) -> LLM:
    """A model folder (config.json + model.safetensors) -> LLM.  config.json picks the architecture."""
    return LLM(load_model(model_dir, dtype=dtype, device=device), max_tokens, max_seqs, use_graphs)


def load_random(
    config: Union[str, Mapping],
    seed: int = 0,
    dtype: str = "bfloat16",
    device: str = "cuda:0",
    max_tokens: Optional[int] = None,
    max_seqs: Optional[int] = None,
    use_graphs: bool = True,
    std: float = 0.02,
    norm_jitter: float = 0.0,
) -> LLM:
    """An LLM with random weights made on the device from a configuration (a dict or a folder with config.json)."""
    cfg = read_config_json(config) if isinstance(config, str) else config
    return LLM(random_model(cfg, seed, dtype, device, std, norm_jitter), max_tokens, max_seqs, use_graphs)
