"""The generation loop above the step function.

One call takes any number of prompts of any lengths.  Prompts are cut into batches
that fit the cache; the prompts of a batch start together in one step, then every
sequence that is still running gets one token per step; a sequence that meets a stop
token, its token budget or the model's position limit leaves the batch (its slot and
pages are given back at once) and the others go on; when a batch has drained the next
one starts in the freed slots.  The reference's single-sequence loop is
`generate_prefilled` (src/model.rs:1714-1763); its server runs the batched form with
one slot per request (src/server.rs:400-453).

Launching ahead: where the engine offers `step_device_tokens`, and every running sequence
will go on unless it has just drawn a stop token, the next step is launched on the tokens
as they lie on the device, before the host has read them.  The host then reads the tokens of
step n while the GPU runs step n + 1, so that launching a step (a graph of a few hundred
kernels) and the loop's own work cost no GPU time.  A sequence that did draw a stop token
has then been stepped once too often: its row of the new logits is dropped and its slot
closed, nothing else changes, and the tokens are the same as without launching ahead.

The loop only needs the four methods of `Engine` and the one of `Sampler` it calls,
so its decisions can be tested with stand-ins that need no GPU.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Union

from ..cache import PAGE_SIZE
from ..errors import StepError
from ..sampling.sampler import SamplingParams, default_seed, sequence_seed
from .engine import StepEntry

STOP_TOKEN = "stop_token"
MAX_NEW_TOKENS = "max_new_tokens"
POSITION_LIMIT = "position_limit"


@dataclass
class GenerationResult:
    tokens: List[int]
    finish_reason: str


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    batches: int = 0
    decode_steps: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    # host time inside the calls of the decode phase (part of decode_seconds): building and
    # launching steps, which the GPU waits for, and sampling, which mostly waits for the GPU
    decode_step_call_seconds: float = 0.0
    decode_sample_call_seconds: float = 0.0


@dataclass
class _Running:
    request: int
    slot: int
    length: int  # positions in the cache
    out: List[int] = field(default_factory=list)
    next_token: int = -1


def plan_batches(prompt_lens: Sequence[int], budgets: Sequence[int], max_positions: int, page_budget: int, max_batch: int) -> List[List[int]]:
    """Cut the requests, in order, into batches whose worst-case page use fits `page_budget`
    and whose size is at most `max_batch`.  budgets[i]: tokens request i may produce.
    A request that cannot fit alone is an error."""
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, n in enumerate(prompt_lens):
        worst = min(n + budgets[i], max_positions)
        pages = (worst + PAGE_SIZE - 1) // PAGE_SIZE
        if pages > page_budget:
            raise StepError(
                f"request {i} may hold {worst} positions ({pages} pages), the cache has {page_budget} pages of {PAGE_SIZE}"
            )
        if cur and (used + pages > page_budget or len(cur) >= max_batch):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += pages
    if cur:
        batches.append(cur)
    return batches


def generate(
    engine,
    sampler,
    prompts: Sequence[Sequence[int]],
    max_new_tokens: Union[int, Sequence[int]],
    params: Optional[SamplingParams] = None,
    stop_token_ids: Optional[Sequence[int]] = None,
    include_stop: bool = False,
    max_batch: Optional[int] = None,
    on_token: Optional[Callable[[int, int], None]] = None,
    stats: Optional[GenerationStats] = None,
    launch_ahead: bool = True,
) -> List[GenerationResult]:
    """Generate up to `max_new_tokens` tokens (one number, or one per prompt) after each prompt;
    results in the prompts' order.

    stop_token_ids: None = the model's own (config.json's eos_token_id).  A stop token ends
    its sequence and is not part of the result (src/model.rs:1749) unless `include_stop`.
    on_token(request index, token) is called for every token as it is produced.
    launch_ahead: see the module's text; False reads every token before the next step starts."""
    params = params or SamplingParams()
    params.validate()
    budgets = [int(max_new_tokens)] * len(prompts) if isinstance(max_new_tokens, int) else [int(b) for b in max_new_tokens]
    if len(budgets) != len(prompts) or any(b < 0 for b in budgets):
        raise StepError(f"max_new_tokens must be >= 0, one number or one per prompt, got {max_new_tokens}")
    stops = set(engine.model.spec.stop_token_ids if stop_token_ids is None else stop_token_ids)
    seed = default_seed() if params.seed is None else params.seed
    max_positions = engine.max_positions
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise StepError(f"prompt {i} is empty")  # as the reference's command line (src/main.rs:294-296)
        if len(p) > max_positions:
            raise StepError(f"prompt {i} has {len(p)} tokens, the model's limit is {max_positions}")
    results: List[Optional[GenerationResult]] = [None] * len(prompts)
    todo = [i for i, b in enumerate(budgets) if b > 0]
    for i, b in enumerate(budgets):
        if b == 0:
            results[i] = GenerationResult([], MAX_NEW_TOKENS)
    limit = max_batch or engine.cache.max_seqs
    batches = [
        [todo[j] for j in group]
        for group in plan_batches(
            [len(prompts[i]) for i in todo], [budgets[i] for i in todo], max_positions, engine.cache.n_pages,
            min(limit, engine.cache.max_seqs),
        )
    ]
    stats = stats if stats is not None else GenerationStats()
    step_ahead = getattr(engine, "step_device_tokens", None) if launch_ahead else None
    # the loop samples from a step's logits before it launches the next step, so it may borrow them
    step_borrowing = getattr(engine, "step_borrowed", engine.step)

    for batch in batches:
        stats.batches += 1
        running: List[_Running] = []
        try:
            note_budget = getattr(engine, "note_budget", None)
            for r in batch:
                running.append(_Running(r, engine.open_sequence(), 0))
                if note_budget is not None:
                    note_budget(running[-1].slot, budgets[r])
            sampler.seed_slots([s.slot for s in running], [sequence_seed(seed, s.request) for s in running])
            t0 = time.perf_counter()
            entries = [StepEntry(s.slot, list(prompts[s.request]), [len(prompts[s.request]) - 1]) for s in running]
            logits = engine.step(entries)
            for s in running:
                s.length = len(prompts[s.request])
                stats.prompt_tokens += s.length
            first = True
            while running:
                t_call = time.perf_counter()
                sampled = sampler.sample(logits, [s.slot for s in running], params)
                begin_fetch = getattr(sampler, "begin_fetch", None)
                pending = begin_fetch(sampled) if begin_fetch is not None else sampled  # the copy goes first
                ahead = None
                if step_ahead is not None and not first and all(
                    len(s.out) + 1 < budgets[s.request] and s.length + 1 <= max_positions for s in running
                ):
                    # nobody ends on this token unless it is a stop token: launch the next step now
                    # (not after the prompt step, whose end is awaited below to time it and to check it)
                    t_step = time.perf_counter()
                    ahead = step_ahead([s.slot for s in running], sampled)
                    stats.decode_step_call_seconds += time.perf_counter() - t_step
                    stats.decode_steps += 1
                tokens = pending.tolist()
                if not first:
                    stats.decode_sample_call_seconds += time.perf_counter() - t_call
                if first:
                    check = getattr(engine, "check_device_status", None)
                    if check is not None:
                        check()  # the prompt step's kernels have finished: did any of them give up?
                    stats.prefill_seconds += time.perf_counter() - t0
                    t0 = time.perf_counter()
                    first = False
                still: List[_Running] = []
                kept_rows: List[int] = []
                for row, (s, tok) in enumerate(zip(running, tokens)):
                    reason = None
                    if tok in stops:
                        reason = STOP_TOKEN
                        if include_stop:
                            s.out.append(tok)
                    else:
                        s.out.append(tok)
                        stats.generated_tokens += 1
                        if on_token is not None:
                            on_token(s.request, tok)
                        if len(s.out) >= budgets[s.request]:
                            reason = MAX_NEW_TOKENS
                        elif s.length + 1 > max_positions:
                            reason = POSITION_LIMIT
                    if reason is None:
                        s.next_token = tok
                        still.append(s)
                        kept_rows.append(row)
                    else:
                        results[s.request] = GenerationResult(s.out, reason)
                        engine.close_sequence(s.slot)
                        s.slot = -1
                n_before = len(running)
                running = still
                if not running:
                    break
                if ahead is not None:
                    logits = ahead if len(kept_rows) == n_before else ahead[kept_rows]
                else:
                    t_call = time.perf_counter()
                    logits = step_borrowing([StepEntry(s.slot, [s.next_token], [0]) for s in running])
                    stats.decode_step_call_seconds += time.perf_counter() - t_call
                    stats.decode_steps += 1
                for s in running:
                    s.length += 1
            stats.decode_seconds += time.perf_counter() - t0
        finally:
            for s in running:
                if s.slot >= 0:
                    engine.close_sequence(s.slot)
    check = getattr(engine, "check_device_status", None)
    if check is not None:
        check()  # one synchronisation per call: a decode kernel that gave up on a wait made its step's tokens invalid
    return results  # type: ignore[return-value]
