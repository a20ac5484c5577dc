"""The step function: one batch of token runs through the model, from the cache.

The reference has three functions for this: `forward` (one token of one
sequence, src/model.rs:1210), `forward_prefill` (n tokens of one sequence,
logits of the last row, src/model.rs:1382) and `Batch::decode_step` (one token
of each of n sequences, src/model.rs:1068); prompts of several sequences are
prefilled one after the other (src/server.rs:400-424).  Here there is one
`Engine.step`: each entry brings the next tokens of one open sequence, any
number of them, the positions come from the cache, and the logits are computed
at the wanted places only (the reference's last-row-only classifier,
src/model.rs:1406-1417).

A step whose entries all bring one token is a decode step; it runs as a CUDA
graph captured per (batch size, page-table width), with the step's integers
(token ids, positions, page tables) copied into fixed device buffers before
the replay, which is the reference's trick of keeping the position in device
memory so that one captured graph serves every position
(src/backend/cuda.rs:1385-1429).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache import PAGE_SIZE, Cache
from ..errors import StepError
from ..kernels import ops
from ..models.model import Model


@dataclass
class StepEntry:
    """The next tokens of the sequence in `slot`, and the indices among them whose logits are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)


@dataclass
class StepContext:
    """What the parts see of a step.  All tensors are int32 on the device.

    tokens[T], tok_seq[T] (index of the token's sequence in the batch), tok_pos[T]
    (position in its sequence), seq_start[S+1] (offsets of the sequences' tokens),
    seq_pos0[S] (positions held before the step), seq_len[S] (positions held after),
    slot_ids[S], rows[W] (packed indices of the tokens whose logits are wanted)."""

    n_tokens: int
    n_seqs: int
    max_q_len: int
    max_kv_len: int
    plan_kv_len: int  # what launch shapes are planned for (>= max_kv_len; fixed per captured graph)
    decode_only: bool
    slots: List[int]
    q_lens: List[int]
    tokens: torch.Tensor
    tok_seq: torch.Tensor
    tok_pos: torch.Tensor
    seq_start: torch.Tensor
    seq_pos0: torch.Tensor
    seq_len: torch.Tensor
    slot_ids: torch.Tensor
    rows: Optional[torch.Tensor]


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class _MetaBuffers:
    """One pinned host buffer and one device buffer holding all integers of a step,
    so that a step costs one host-to-device copy.  The buffers grow on demand; the
    host side is not refilled before the previous copy out of it has finished."""

    def __init__(self, device: torch.device):
        self.device = device
        self.capacity = 0
        self.host = self.host_np = self.dev = None
        self.sizes: List[int] = []
        self.offsets: List[int] = []
        self.widths: Tuple[int, ...] = ()
        self.total = 0
        self._copied: Optional[torch.cuda.Event] = None

    def layout(self, T: int, S: int, W: int, widths: Sequence[int]) -> None:
        self.widths = tuple(widths)
        self.sizes = [T, T, T, S + 1, S, S, S, W] + [S * w for w in widths]
        self.offsets, total = [], 0
        for n in self.sizes:
            self.offsets.append(total)
            total += _pad4(max(n, 1))
        self.total = total
        self.wait_for_copy()
        if total > self.capacity:
            self.capacity = max(total, 2 * self.capacity)
            pin = self.device.type == "cuda"
            self.host = torch.zeros(self.capacity, dtype=torch.int32, pin_memory=pin)
            self.host_np = self.host.numpy()
            self.dev = torch.zeros(self.capacity, dtype=torch.int32, device=self.device)

    def wait_for_copy(self) -> None:
        """The host side may be rewritten once the last copy out of it has finished."""
        if self._copied is not None:
            self._copied.synchronize()

    def host_part(self, i: int) -> np.ndarray:
        return self.host_np[self.offsets[i] : self.offsets[i] + self.sizes[i]]

    def dev_part(self, i: int) -> torch.Tensor:
        return self.dev[self.offsets[i] : self.offsets[i] + self.sizes[i]]

    def upload(self) -> None:
        self.dev[: self.total].copy_(self.host[: self.total], non_blocking=True)
        if self.device.type == "cuda":
            if self._copied is None:
                self._copied = torch.cuda.Event()
            self._copied.record()


class _DecodeGraph:
    def __init__(self):
        self.meta: Optional[_MetaBuffers] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.warm = 0
        self.launches = 0  # kernels of this library inside the captured graph
        self.members = None  # the slots, in order, whose numbers and page tables the device buffers hold


class Engine:
    """A model, its cache and the step function.

    max_tokens: positions the cache can hold at once (each sequence rounded up to 64).
    max_seqs: sequences that can be open at once (default: one per page, at most 256).
    use_graphs: replay decode steps as CUDA graphs."""

    def __init__(self, model: Model, max_tokens: int, max_seqs: Optional[int] = None, use_graphs: bool = True):
        self.model = model
        self.rt = model.rt
        if max_seqs is None:
            max_seqs = max(1, min((max_tokens + PAGE_SIZE - 1) // PAGE_SIZE, 256))
        self.cache: Cache = model.new_cache(max_tokens, max_seqs)
        self.vocab_size = model.spec.vocab_size
        self.max_positions = model.spec.max_positions
        self.use_graphs = use_graphs and self.rt.device.type == "cuda"
        self._graphs: Dict[Tuple[int, int], _DecodeGraph] = {}
        self._meta = _MetaBuffers(self.rt.device)
        self.uploads = 0  # host-to-device copies of step integers so far (a replayed decode step may need none)
        self.upload_bytes = 0

    # ------------------------------------------------------------------ sequences
    def open_sequence(self) -> int:
        return self.cache.open_sequence()

    def close_sequence(self, slot: int) -> None:
        self.cache.close_sequence(slot)

    def note_budget(self, slot: int, max_new: int) -> None:
        """Write into the slot's record on the device how many tokens its sequence may decode."""
        self.cache.set_budget(slot, max_new)

    def sequence_record(self, slot: int) -> dict:
        """The slot's record as the device holds it: positions held, tokens decoded, budget, open (synchronises)."""
        return self.cache.record(slot)

    def check_device_status(self) -> None:
        """Raise if a kernel with bounded waits gave up since the last check.  Synchronises the device."""
        ops.tc_status_check()

    # ------------------------------------------------------------------ the step
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"the entry of slot {e.slot} brings no token")
            have = self.cache.length(e.slot)  # raises CacheError for a slot that is not open
            if have + n > self.max_positions:
                raise StepError(
                    f"slot {e.slot} would reach position {have + n}, the model's limit is {self.max_positions}"
                )
            for t in e.tokens:
                if not 0 <= int(t) < self.vocab_size:
                    raise StepError(f"token id {t} of slot {e.slot} is outside the vocabulary of {self.vocab_size}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"slot {e.slot} wants logits at index {w} of {n} tokens")

    def _fill_meta(self, meta: _MetaBuffers, entries: Sequence[StepEntry], pos0: List[int], rows: List[int]) -> None:
        S = len(entries)
        tokens, tok_seq, tok_pos = meta.host_part(0), meta.host_part(1), meta.host_part(2)
        seq_start, seq_pos0, seq_len, slot_ids = meta.host_part(3), meta.host_part(4), meta.host_part(5), meta.host_part(6)
        at = 0
        for i, e in enumerate(entries):
            n = len(e.tokens)
            tokens[at : at + n] = e.tokens
            tok_seq[at : at + n] = i
            tok_pos[at : at + n] = np.arange(pos0[i], pos0[i] + n, dtype=np.int32)
            seq_start[i] = at
            seq_pos0[i] = pos0[i]
            seq_len[i] = pos0[i] + n
            slot_ids[i] = e.slot
            at += n
        seq_start[S] = at
        if rows:
            meta.host_part(7)[: len(rows)] = rows
        slots = [e.slot for e in entries]
        for g, width in enumerate(meta.widths):
            meta.host_part(8 + g)[:] = self.cache.block_table(g, slots, width).reshape(-1)

    def _context(self, meta: _MetaBuffers, entries, pos0, n_rows: int, plan_kv_len: int) -> Tuple[StepContext, List[torch.Tensor]]:
        q_lens = [len(e.tokens) for e in entries]
        S = len(entries)
        step = StepContext(
            n_tokens=sum(q_lens),
            n_seqs=S,
            max_q_len=max(q_lens),
            max_kv_len=max(p + q for p, q in zip(pos0, q_lens)),
            plan_kv_len=plan_kv_len,
            decode_only=all(q == 1 for q in q_lens),
            slots=[e.slot for e in entries],
            q_lens=q_lens,
            tokens=meta.dev_part(0),
            tok_seq=meta.dev_part(1),
            tok_pos=meta.dev_part(2),
            seq_start=meta.dev_part(3),
            seq_pos0=meta.dev_part(4),
            seq_len=meta.dev_part(5),
            slot_ids=meta.dev_part(6),
            rows=meta.dev_part(7)[:n_rows] if n_rows else None,
        )
        tables = [meta.dev_part(8 + g).view(S, w) for g, w in enumerate(meta.widths)]
        return step, tables

    def step(self, entries: Sequence[StepEntry], borrow: bool = False) -> torch.Tensor:
        """Run the entries' tokens; returns float32 logits [wanted, vocab] on the device,
        in the order of the entries and of each entry's `want`.

        The result is the caller's to keep.  borrow=True skips the copy that makes it so: a decode
        step that was replayed as a CUDA graph then returns the graph's own output buffer, which
        the next decode step of the same batch size overwrites; a caller that has consumed the
        logits before its next call (in stream order: sampling from them is enough) may ask for that."""
        if self.use_graphs and entries and all(len(e.tokens) == 1 for e in entries):
            logits = self._decode_graph_step(entries)
            return logits if borrow else logits.clone()
        self._validate(entries)
        slots = [e.slot for e in entries]
        q_lens = [len(e.tokens) for e in entries]
        pos0 = [self.cache.length(s) for s in slots]
        self.cache.reserve(slots, q_lens)
        rows: List[int] = []
        at = 0
        for e in entries:
            rows.extend(at + int(w) for w in e.want)
            at += len(e.tokens)
        T, S = sum(q_lens), len(entries)
        widths = tuple(self.cache.table_width(slots) for _ in self.cache.kv_groups)
        meta = self._meta
        meta.layout(T, S, len(rows), widths)
        self._fill_meta(meta, entries, pos0, rows)
        meta.upload()
        self.uploads += 1
        self.upload_bytes += 4 * meta.total
        step, tables = self._context(meta, entries, pos0, len(rows), max(p + q for p, q in zip(pos0, q_lens)))
        logits = self.model.forward(step, self.cache, tables)
        if self.rt.device.type == "cuda":
            ops.seq_set_len(self.cache.seq_records, step.slot_ids, step.seq_len)  # the records follow a step whose positions the host gave
        self.cache.commit(slots, q_lens)
        return logits

    def step_borrowed(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """`step(entries, borrow=True)`, for loops that consume a step's logits before their next call."""
        return self.step(entries, borrow=True)

    # ------------------------------------------------------------------ decode through a graph
    def step_device_tokens(self, slots: Sequence[int], tokens: torch.Tensor) -> torch.Tensor:
        """One token for each of `slots`, taken from `tokens` (int32 [len(slots)] on the device, for
        instance what the sampler just wrote) without the host ever seeing them; logits for every
        slot.  The generation loop uses it to launch a step before it has read the previous step's
        tokens, so that launching overlaps the GPU's work.

        The logits are borrowed (see `step`): they are the replayed graph's output buffer and hold
        this step's values only until the next decode step of the same batch size is launched."""
        if tokens.dtype != torch.int32 or tokens.device != self.rt.device or tuple(tokens.shape) != (len(slots),):
            raise StepError(f"step_device_tokens wants int32 [{len(slots)}] on {self.rt.device}, got {tokens.dtype} {tuple(tokens.shape)} on {tokens.device}")
        entries = [StepEntry(int(s), [0], [0]) for s in slots]
        if not self.use_graphs:
            for e, t in zip(entries, tokens.tolist()):
                e.tokens[0] = int(t)
            return self.step(entries)
        return self._decode_graph_step(entries, tokens)

    def _decode_graph_step(self, entries, device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """A step whose entries all bring one token: checks, cache bookkeeping and the step's integers
        are done with array operations, the kernels are one graph replay.  device_tokens: the token
        ids are copied from this device tensor into the step's buffer after the host's upload."""
        S = len(entries)
        slots = np.fromiter((e.slot for e in entries), dtype=np.intp, count=S)
        toks = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=S)
        if len(set(slots.tolist())) != S:
            raise StepError(f"a slot appears twice in one step: {slots.tolist()}")
        pos0 = self.cache.lengths(slots)  # raises CacheError for a slot that is not open
        if ((toks < 0) | (toks >= self.vocab_size)).any():
            bad = toks[(toks < 0) | (toks >= self.vocab_size)][0]
            raise StepError(f"token id {int(bad)} is outside the vocabulary of {self.vocab_size}")
        if (pos0 + 1 > self.max_positions).any():
            raise StepError(f"a sequence would pass the model's limit of {self.max_positions} positions")
        rows: List[int] = []
        for i, e in enumerate(entries):
            if len(e.want):
                if len(e.want) != 1 or int(e.want[0]) != 0:
                    raise StepError(f"slot {e.slot} wants logits at {list(e.want)} of 1 token")
                rows.append(i)
        took_page = self.cache.reserve_one_each(slots, pos0)
        need_width = (int(pos0.max()) + PAGE_SIZE) // PAGE_SIZE
        width = 4
        while width < need_width:
            width *= 2
        key = (S, width)
        g = self._graphs.get(key)
        if g is None:
            g = _DecodeGraph()
            g.meta = _MetaBuffers(self.rt.device)
            g.meta.layout(S, S, S, tuple(width for _ in self.cache.kv_groups))
            ar = np.arange(S + 1, dtype=np.int32)
            g.meta.host_part(1)[:] = ar[:S]  # each token is its own sequence
            g.meta.host_part(3)[:] = ar
            g.meta.host_part(7)[:] = ar[:S]
            g.host = [g.meta.host_part(i) for i in range(8 + len(self.cache.kv_groups))]
            self._graphs[key] = g
        # What the device buffers of this graph have to be told: the tokens, unless they lie on the device already;
        # the slots and their page tables, unless they are the ones of this graph's last step and no sequence
        # took a page (a window group also gives pages back, so its tables are sent every time).  The positions
        # are never sent: the step's first kernel takes them from the records on the device.
        members = tuple(slots.tolist())
        if g.graph is None or device_tokens is None or g.members != members or took_page or self.cache.has_window_groups():
            g.meta.wait_for_copy()
            h = g.host
            h[0][:] = toks
            h[6][:] = slots
            for gi in range(len(self.cache.kv_groups)):
                h[8 + gi][:] = self.cache.block_table(gi, slots, width).reshape(-1)
            g.meta.upload()
            self.uploads += 1
            self.upload_bytes += 4 * g.meta.total
            g.members = members
        if device_tokens is not None:
            g.meta.dev_part(0).copy_(device_tokens, non_blocking=True)
        meta = g.meta
        begin = lambda: ops.seq_begin_decode(self.cache.seq_records, meta.dev_part(6), meta.dev_part(2), meta.dev_part(4), meta.dev_part(5))  # noqa: E731
        if g.graph is None:
            pos_list = pos0.tolist()
            step, tables = self._context(g.meta, entries, pos_list, S, width * PAGE_SIZE)
            if g.warm < 1:
                # first use of this shape: run it plainly, which also sizes the workspaces
                g.warm += 1
                begin()
                logits = self.model.forward(step, self.cache, tables)
            else:
                torch.cuda.synchronize(self.rt.device)
                graph = torch.cuda.CUDAGraph()
                before = ops.launch_count()
                with torch.cuda.graph(graph):
                    begin()
                    g.logits = self.model.forward(step, self.cache, tables)
                g.launches = ops.launch_count() - before
                g.graph = graph
                graph.replay()
                logits = g.logits
        else:
            g.graph.replay()
            ops.add_launches(g.launches)
            logits = g.logits
        self.cache.commit_one_each(slots)
        if len(rows) == S:
            return logits
        if not rows:
            return logits[:0]
        return logits[torch.tensor(rows, dtype=torch.long, device=logits.device)]
