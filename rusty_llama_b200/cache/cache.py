"""The cache: per-sequence storage that outlives a step.

What the reference keeps per sequence is a flat K/V array grown in 256-position
pages plus scattered fixed-size records: the position, the sampler's random
state (src/model.rs:722-834, src/server.rs:286-296).  Its shared budget
`KvPagePool` only counts cells for admission (src/model.rs:646-698).  Here the
pages are real: storage is a pool of pages of 64 positions, a sequence holds a
list of pages per group of layers, and the attention kernels find a position
through that list.  A sequence therefore costs what it holds, rounded up to 64,
whatever the lengths of the others.

Layers are grouped by what they need.  All runs of the schedule that need the
same (kv heads, head size, window) share one group: one tensor
[runs, pages, kv heads, 64, head size] for keys, one for values, one page list
per sequence.  A group with a window gives pages back as they fall out of the
window; a group of fixed-size state has one record per (run, sequence), zeroed
when a sequence opens.  A sequence is known by its slot, an index that is
handed out by `open_sequence`, given back by `close_sequence` and then used
again.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..errors import CacheError
from ..parts.base import KVNeed, StateNeed

PAGE_SIZE = 64


class PagePool:
    """Which pages of a group are free.  Knows nothing about tensors."""

    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, got {n_pages}")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))  # pop() hands out 0 first
        self._held = np.zeros(n_pages, dtype=bool)

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"out of cache pages: all {self.n_pages} pages of {PAGE_SIZE} positions are held")
        page = self._free.pop()
        if self._held[page]:
            raise CacheError(f"page {page} was on the free list while held")
        self._held[page] = True
        return page

    def give_back(self, page: int) -> None:
        if not 0 <= page < self.n_pages:
            raise CacheError(f"page {page} does not exist")
        if not self._held[page]:
            raise CacheError(f"page {page} is given back twice")
        self._held[page] = False
        self._free.append(page)


@dataclass
class KVView:
    """One run's keys and values, with the page lists of the step's sequences."""

    k_pages: torch.Tensor  # [pages, kv heads, PAGE_SIZE, head size]
    v_pages: torch.Tensor
    block_table: Optional[torch.Tensor]  # int32 [S, width] on the device, set per step
    window: int


@dataclass
class StateView:
    """One run's fixed-size records: state[slot] is the record of the sequence in that slot."""

    state: torch.Tensor  # [max sequences, *shape]


class KVGroup:
    def __init__(self, need: KVNeed, runs: List[int], n_pages: int, dtype: torch.dtype, device: torch.device, max_seqs: int = 1):
        self.need = need
        self.runs = list(runs)
        self.pool = PagePool(n_pages)
        shape = (len(runs), n_pages, need.num_kv_heads, PAGE_SIZE, need.head_dim)
        dtype = need.dtype or dtype  # a need may name its own storage type; else the run's
        # zero-filled once: a page that was never written holds finite values, which the
        # attention kernels rely on when they multiply masked scores by unread rows
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.pages: Dict[int, List[int]] = {}  # slot -> page id per page index (-1: given back)
        self.first_held: Dict[int, int] = {}  # slot -> lowest page index still held
        # the same page lists as one matrix [slot, page index] (0 where nothing is held), kept in
        # step with `pages` so that a step's block table is one indexing operation
        self.table = np.zeros((max_seqs, 8), dtype=np.int32)

    def _set(self, slot: int, index: int, page: int) -> None:
        if index >= self.table.shape[1]:
            grown = np.zeros((self.table.shape[0], max(2 * self.table.shape[1], index + 1)), dtype=np.int32)
            grown[:, : self.table.shape[1]] = self.table
            self.table = grown
        self.table[slot, index] = max(page, 0)

    def bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()

    def first_needed_page(self, next_pos: int) -> int:
        """Lowest page index that a query at `next_pos` or later can still read."""
        if not self.need.window:
            return 0
        return max(0, next_pos - self.need.window + 1) // PAGE_SIZE


class StateGroup:
    def __init__(self, need: StateNeed, runs: List[int], max_seqs: int, device: torch.device):
        self.need = need
        self.runs = list(runs)
        self.state = torch.zeros((len(runs), max_seqs) + tuple(need.shape), dtype=need.dtype, device=device)

    def bytes(self) -> int:
        return self.state.numel() * self.state.element_size()


class Cache:
    """needs: for each run of the schedule that owns cache storage, (run index, KVNeed | StateNeed).
    max_tokens: positions that can be held at once, each sequence rounded up to PAGE_SIZE.
    max_seqs: sequences that can be open at once."""

    def __init__(
        self,
        needs: Sequence[Tuple[int, object]],
        max_tokens: int,
        max_seqs: int,
        dtype: torch.dtype,
        device,
    ):
        if max_tokens <= 0 or max_seqs <= 0:
            raise CacheError(f"a cache needs positive sizes, got max_tokens={max_tokens}, max_seqs={max_seqs}")
        self.device = torch.device(device)
        self.dtype = dtype
        self.n_pages = (max_tokens + PAGE_SIZE - 1) // PAGE_SIZE
        self.max_tokens = self.n_pages * PAGE_SIZE
        self.max_seqs = max_seqs
        by_need: Dict[object, List[int]] = {}
        for run, need in needs:
            if not isinstance(need, (KVNeed, StateNeed)):
                raise CacheError(f"run {run} asks for {need!r}, which is neither a KVNeed nor a StateNeed")
            by_need.setdefault(need, []).append(run)
        if self.device.type == "cuda":
            # say so before allocating, with the numbers, instead of running out of memory half-way
            asked = 0
            for need, runs in by_need.items():
                if isinstance(need, KVNeed):
                    size = torch.empty((), dtype=need.dtype or dtype).element_size()
                    asked += 2 * len(runs) * self.n_pages * need.num_kv_heads * PAGE_SIZE * need.head_dim * size
                else:
                    n = torch.empty((), dtype=need.dtype).element_size() * max_seqs * len(runs)
                    for s in need.shape:
                        n *= s
                    asked += n
            # free on the device, plus what torch's allocator holds without using it (it hands that out first)
            free = torch.cuda.mem_get_info(self.device)[0] + torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)
            if asked > free:
                raise CacheError(
                    f"a cache of {self.max_tokens} positions needs {asked / 2**30:.1f} GiB, the device has {free / 2**30:.1f} GiB free: "
                    f"ask for fewer positions (max_tokens)")
        self.kv_groups: List[KVGroup] = []
        self.state_groups: List[StateGroup] = []
        self._where: Dict[int, Tuple[str, int, int]] = {}  # run -> (family, group index, index in group)
        for need, runs in by_need.items():
            if isinstance(need, KVNeed):
                self.kv_groups.append(KVGroup(need, runs, self.n_pages, dtype, self.device, max_seqs))
                gi = len(self.kv_groups) - 1
                for j, run in enumerate(runs):
                    self._where[run] = ("kv", gi, j)
            else:
                self.state_groups.append(StateGroup(need, runs, max_seqs, self.device))
                gi = len(self.state_groups) - 1
                for j, run in enumerate(runs):
                    self._where[run] = ("state", gi, j)
        # Fixed-size record per sequence slot, on the device: positions held, tokens decoded, the most it may decode,
        # flags (bit 0: open).  The host keeps its own copy of the lengths for its bookkeeping (`_length`); a decode
        # step's kernels take theirs from here (`ops.seq_begin_decode`), so a replayed graph needs no upload of them.
        self.seq_records = torch.zeros((max_seqs, 4), dtype=torch.int32, device=self.device)
        self._free_slots: List[int] = list(range(max_seqs - 1, -1, -1))
        self._record_open = torch.tensor([0, 0, 0, 1], dtype=torch.int32, device=self.device)
        self._open = np.zeros(max_seqs, dtype=bool)
        self._length = np.zeros(max_seqs, dtype=np.int64)

    # ------------------------------------------------------------------ sequences
    @property
    def n_open(self) -> int:
        return int(self._open.sum())

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.kv_groups) + sum(g.bytes() for g in self.state_groups)

    def open_sequence(self) -> int:
        if not self._free_slots:
            raise CacheError(f"all {self.max_seqs} sequence slots are in use")
        slot = self._free_slots.pop()
        if self._open[slot]:
            raise CacheError(f"slot {slot} was on the free list while open")
        self._open[slot] = True
        self._length[slot] = 0
        for g in self.kv_groups:
            g.pages[slot] = []
            g.first_held[slot] = 0
            g.table[slot, :] = 0
        for g in self.state_groups:
            g.state[:, slot].zero_()
        self.seq_records[slot] = self._record_open  # nothing held, nothing decoded, no budget named, open
        return slot

    def set_budget(self, slot: int, max_new: int) -> None:
        """Note in the slot's record how many tokens its sequence may decode (0: no limit named)."""
        self._check_open(slot)
        self.seq_records[slot, 2] = int(max_new)

    def close_sequence(self, slot: int) -> None:
        self._check_open(slot)
        for g in self.kv_groups:
            for page in g.pages.pop(slot):
                if page >= 0:
                    g.pool.give_back(page)
            g.first_held.pop(slot)
        self._open[slot] = False
        self._length[slot] = 0
        self._free_slots.append(slot)
        self.seq_records[slot, 3] = 0  # closed; what it held and decoded stays readable until the slot opens again

    def _check_open(self, slot: int) -> None:
        if not (isinstance(slot, (int, np.integer)) and 0 <= slot < self.max_seqs):
            raise CacheError(f"slot {slot!r} does not exist")
        if not self._open[slot]:
            raise CacheError(f"slot {slot} is not open (never opened, or closed already)")

    def length(self, slot: int) -> int:
        self._check_open(slot)
        return int(self._length[slot])

    def pages_free(self) -> int:
        return min((g.pool.n_free for g in self.kv_groups), default=self.n_pages)

    # ------------------------------------------------------------------ a step
    def reserve(self, slots: Sequence[int], q_lens: Sequence[int]) -> None:
        """Make room for q_lens[i] more positions of slots[i] in every group, or change nothing and raise."""
        if len(set(slots)) != len(slots):
            raise CacheError(f"a slot appears twice in one step: {list(slots)}")
        for slot in slots:
            self._check_open(slot)
        taken: List[Tuple[KVGroup, int]] = []
        try:
            for g in self.kv_groups:
                for slot, q in zip(slots, q_lens):
                    have = g.pages[slot]
                    need_pages = (int(self._length[slot]) + q + PAGE_SIZE - 1) // PAGE_SIZE
                    while len(have) < need_pages:
                        page = g.pool.take()
                        have.append(page)
                        g._set(slot, len(have) - 1, page)
                        taken.append((g, slot))
        except CacheError:
            for g, slot in reversed(taken):
                g._set(slot, len(g.pages[slot]) - 1, 0)
                g.pool.give_back(g.pages[slot].pop())
            raise

    def commit(self, slots: Sequence[int], q_lens: Sequence[int]) -> None:
        """The step ran: lengths grow, pages that no later query can read go back to their pool."""
        for slot, q in zip(slots, q_lens):
            self._length[slot] += q
        for g in self.kv_groups:
            if not g.need.window:
                continue
            for slot in slots:
                keep_from = g.first_needed_page(int(self._length[slot]))
                have = g.pages[slot]
                for idx in range(g.first_held[slot], min(keep_from, len(have))):
                    if have[idx] >= 0:
                        g.pool.give_back(have[idx])
                        have[idx] = -1
                        g._set(slot, idx, 0)
                g.first_held[slot] = max(g.first_held[slot], min(keep_from, len(have)))

    def table_width(self, slots: Sequence[int]) -> int:
        return max((len(g.pages[s]) for g in self.kv_groups for s in slots), default=1) or 1

    def lengths(self, slots: np.ndarray) -> np.ndarray:
        """Positions held by each of `slots` (an integer array); raises if one is not open."""
        if slots.size and (slots.min() < 0 or slots.max() >= self.max_seqs or not self._open[slots].all()):
            bad = [int(s) for s in slots if not (0 <= s < self.max_seqs) or not self._open[s]]
            raise CacheError(f"slots {bad} are not open (never opened, or closed already)")
        return self._length[slots]

    def has_window_groups(self) -> bool:
        return any(g.need.window for g in self.kv_groups)

    def reserve_one_each(self, slots: Sequence[int], lengths: np.ndarray) -> bool:
        """`reserve(slots, [1] * len(slots))` for the common decode step: a page is taken only by the
        sequences that stand at a page boundary.  Returns whether any page list changed."""
        at_boundary = [int(s) for s, n in zip(slots, lengths) if n % PAGE_SIZE == 0]
        if at_boundary:
            self.reserve(at_boundary, [1] * len(at_boundary))
        return bool(at_boundary)

    def record(self, slot: int) -> dict:
        """The slot's record as the device holds it (synchronises): for tests and for looking at a run."""
        held, decoded, max_new, flags = self.seq_records[slot].tolist()
        return {"len": held, "decoded": decoded, "max_new": max_new, "open": bool(flags & 1)}

    def commit_one_each(self, slots: np.ndarray) -> None:
        if self.has_window_groups():
            self.commit([int(s) for s in slots], [1] * len(slots))
        else:
            self._length[slots] += 1

    def block_table(self, group_index: int, slots: Sequence[int], width: int) -> np.ndarray:
        """int32 [len(slots), width]: page id of page index j of each sequence; unheld entries are 0."""
        g = self.kv_groups[group_index]
        have = g.table.shape[1]
        if width <= have:
            return g.table[np.asarray(slots, dtype=np.intp), :width]
        table = np.zeros((len(slots), width), dtype=np.int32)
        table[:, :have] = g.table[np.asarray(slots, dtype=np.intp)]
        return table

    # ------------------------------------------------------------------ views
    def where(self, run: int) -> Tuple[str, int, int]:
        try:
            return self._where[run]
        except KeyError:
            raise CacheError(f"run {run} of the schedule owns no cache storage") from None

    def view(self, run: int, tables: Optional[Sequence[torch.Tensor]] = None):
        """The storage of one run.  tables[g]: this step's device block table of kv group g."""
        family, gi, j = self.where(run)
        if family == "kv":
            g = self.kv_groups[gi]
            return KVView(g.k[j], g.v[j], None if tables is None else tables[gi], g.need.window)
        return StateView(self.state_groups[gi].state[j])

    def check_consistent(self) -> None:
        """Every page is either free or held by exactly one open sequence; raises otherwise."""
        for gi, g in enumerate(self.kv_groups):
            seen = np.zeros(g.pool.n_pages, dtype=np.int64)
            for slot, pages in g.pages.items():
                if not self._open[slot]:
                    raise CacheError(f"group {gi}: closed slot {slot} still has a page list")
                for p in pages:
                    if p >= 0:
                        seen[p] += 1
            if (seen > 1).any():
                raise CacheError(f"group {gi}: pages {np.nonzero(seen > 1)[0].tolist()} are held twice")
            free = np.zeros(g.pool.n_pages, dtype=np.int64)
            for p in g.pool._free:
                free[p] += 1
            if (free > 1).any():
                raise CacheError(f"group {gi}: pages {np.nonzero(free > 1)[0].tolist()} are on the free list twice")
            if ((seen + free) != 1).any():
                bad = np.nonzero((seen + free) != 1)[0].tolist()
                raise CacheError(f"group {gi}: pages {bad} are lost or both free and held")
        open_slots = set(np.nonzero(self._open)[0].tolist())
        free_slots = set(self._free_slots)
        if len(free_slots) != len(self._free_slots) or open_slots & free_slots or len(open_slots | free_slots) != self.max_seqs:
            raise CacheError("sequence slots are lost, free twice, or both free and open")
