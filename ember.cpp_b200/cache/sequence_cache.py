"""The cache: a slot for each live sequence, keys and values for each layer in pages of 64
positions, and per-sequence state of fixed size beside them.

ember.cpp's interpreter keeps, per block, keys and values as [max_len][kv_heads][head_dim] for
its one sequence (graph_ir.h:310, 462), a window per layer where a model has one
(graph_ir.h:318-322), and fixed-size recurrent state per layer in a separate region
(graph_ir.h:343-369, 506-515); its llama path has per-sequence lengths for a batch
(model.h:148-160).  Here:

* A *slot* belongs to one sequence from `open()` to `close()`: its length, its pages in every
  group, and its row in every state tensor.  Closed slots are used again.
* Layers with the same need (all keys, or a window of them; head count; head size) form a *group*
  with storage of its own: per application of the schedule one K and one V tensor of shape
  [pages, kv_heads, 64, head_dim], and one pool of page numbers shared by the group's layers.  A
  sequence holds ceil(length / 64) pages of a full group; a window group gives back the pages that
  lie wholly before the window.
* `max_tokens` sizes every group's pool: the most positions that live sequences hold at any time,
  each sequence's count rounded up to a multiple of 64.
* State tensors are [slots, *shape] float32 per application that asks for one, set to the part's
  initial value when a slot is opened.

All bookkeeping is on the host.  `reserve` checks a whole step before it changes anything.
"""
from __future__ import annotations

import numpy as np
import torch

from ..parts.base import CacheNeed, StateNeed
from .allocator import Pool, PoolError

PAGE = 64


class CacheError(RuntimeError):
    pass


class CacheGroup:
    """Storage of the applications that share one CacheNeed."""

    def __init__(self, need: CacheNeed, apps: list[int], n_pages: int, n_slots: int, dtype, device):
        self.need, self.apps = need, list(apps)
        self.pages = Pool(n_pages, "page")
        shape = (n_pages, need.kv_heads, PAGE, need.head_dim)
        self.k = [torch.zeros(shape, dtype=dtype, device=device) for _ in apps]
        self.v = [torch.zeros(shape, dtype=dtype, device=device) for _ in apps]
        # per slot: page number of each 64-position block, -1 where none is held
        self.held: list[list[int]] = [[] for _ in range(n_slots)]

    def first_needed_block(self, next_position: int) -> int:
        """The first block that a query at `next_position` can still read."""
        if self.need.kind != "window":
            return 0
        return max(0, next_position - self.need.window + 1) // PAGE

    def pages_missing(self, slot: int, start: int, n_new: int) -> int:
        blocks = -(-(start + n_new) // PAGE)
        have = self.held[slot]
        first = self.first_needed_block(start)
        return sum(1 for b in range(first, blocks) if b >= len(have) or have[b] < 0)

    def ensure(self, slot: int, start: int, n_new: int) -> list[int]:
        """Takes the pages that positions start .. start + n_new - 1 need; returns the blocks (64-position
        runs of the sequence) whose page is new."""
        blocks = -(-(start + n_new) // PAGE)
        have = self.held[slot]
        first = self.first_needed_block(start)
        while len(have) < blocks:
            have.append(-1)
        fresh = []
        for b in range(first, blocks):
            if have[b] < 0:
                have[b] = self.pages.take()
                fresh.append(b)
        return fresh

    def trim(self, slot: int, length: int) -> None:
        """Gives back what no later query can read (window groups), or what lies past `length`."""
        have = self.held[slot]
        for b in range(min(self.first_needed_block(length), len(have))):
            if have[b] >= 0:
                self.pages.give_back(have[b])
                have[b] = -1
        blocks = -(-length // PAGE)
        while len(have) > blocks:
            p = have.pop()
            if p >= 0:
                self.pages.give_back(p)

    def release(self, slot: int) -> None:
        for p in self.held[slot]:
            if p >= 0:
                self.pages.give_back(p)
        self.held[slot] = []

    def table(self, slots, width: int) -> np.ndarray:
        out = np.full((len(slots), width), -1, dtype=np.int32)
        for i, s in enumerate(slots):
            if s >= 0:
                row = self.held[s]
                out[i, :len(row)] = row
        return out


class CacheView:
    """What one application's mixer sees of its group."""

    def __init__(self, group_index: int, group: CacheGroup, local: int):
        self.group_index = group_index
        self.k, self.v = group.k[local], group.v[local]
        # the storage of the application that runs next from this group (the first one after the last):
        # a kernel may warm it while it reads this one
        n = len(group.k)
        self.following = (group.k[(local + 1) % n], group.v[(local + 1) % n]) if n > 1 else None
        self.kv_heads, self.head_dim = group.need.kv_heads, group.need.head_dim
        self.window = group.need.window if group.need.kind == "window" else 0


class SequenceCache:
    def __init__(self, needs: list[tuple[CacheNeed | None, StateNeed | None]], cache_of: list[int | None],
                 max_tokens: int, max_positions: int | None, dtype, device, max_slots: int | None = None):
        if max_tokens <= 0:
            raise CacheError(f"max_tokens = {max_tokens} must be positive")
        self.n_pages = -(-int(max_tokens) // PAGE)
        self.max_tokens = self.n_pages * PAGE
        self.max_positions = max_positions
        longest = self.max_tokens if max_positions is None else min(self.max_tokens, -(-max_positions // PAGE) * PAGE)
        self.max_blocks = longest // PAGE
        self.n_slots = self.n_pages if max_slots is None else max(1, min(int(max_slots), self.n_pages))
        self.slots = Pool(self.n_slots, "slot")
        self.lengths = [0] * self.n_slots
        self.dtype, self.device = dtype, device

        keys: dict[CacheNeed, list[int]] = {}
        for i, (need, _) in enumerate(needs):
            if need is not None and cache_of[i] is None:   # an entry that reads another's cache has none of its own
                keys.setdefault(need, []).append(i)
        self.groups = [CacheGroup(need, apps, self.n_pages, self.n_slots, dtype, device) for need, apps in keys.items()]
        self.views: list[CacheView | None] = [None] * len(needs)
        for gi, g in enumerate(self.groups):
            for local, app in enumerate(g.apps):
                self.views[app] = CacheView(gi, g, local)
        self.writes = [needs[i][0] is not None and cache_of[i] is None for i in range(len(needs))]
        for i, src in enumerate(cache_of):
            if src is not None:
                if self.views[src] is None:
                    raise CacheError(f"schedule entry {i} reads the cache of entry {src}, which has none")
                self.views[i] = self.views[src]
                self.writes[i] = False
        self.state_needs = [s for _, s in needs]

        def make(need: StateNeed):
            if need.dtype not in ("float32", "int32"):
                raise CacheError(f"per-sequence state of type {need.dtype!r}: float32 or int32")
            return torch.full((self.n_slots, *need.shape), need.init, dtype=getattr(torch, need.dtype), device=device)

        # per application: None, one tensor [slots, *shape], or (a mixer with several) a dict of them by name
        self.states = [None if s is None else ({k: make(v) for k, v in s.items()} if isinstance(s, dict) else make(s))
                       for s in self.state_needs]

    # ------------------------------------------------------------------ slots
    def open(self) -> int:
        try:
            slot = self.slots.take()
        except PoolError as e:
            raise CacheError(str(e)) from None
        self.lengths[slot] = 0
        for need, state in zip(self.state_needs, self.states):
            if isinstance(state, dict):
                for name, t in state.items():
                    t[slot].fill_(need[name].init)
            elif state is not None:
                state[slot].fill_(need.init)
        return slot

    def close(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is closed but is not open")
        for g in self.groups:
            g.release(slot)
        self.lengths[slot] = 0
        self.slots.give_back(slot)

    def length(self, slot: int) -> int:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not open")
        return self.lengths[slot]

    # ------------------------------------------------------------------ a step's storage
    def reserve(self, step: list[tuple[int, int]]) -> list[list[tuple[int, int]]]:
        """`step`: (slot, number of new positions) per sequence.  Checks everything, then takes
        the pages; on an error nothing has changed.

        Returns, per group and per sequence of the step, (page, first row) of a tail to clear, or
        (-1, 0): pages are not cleared when they change hands (ember.cpp does not clear its cache
        between requests either: rows are written before they are read, api.cpp:943-944), so a page
        that is new to a sequence holds whatever its last owner left, possibly NaN or Inf.  Kernels
        that load whole pages multiply a probability of exactly zero with the rows past a
        sequence's end, and zero times NaN is NaN.  So when the page that will hold a sequence's
        last position after this step is new to it, the rows of that page past the step's end are
        cleared before the step runs (`tails`); every other row of a new page is written by the
        step itself.  A held page then holds finite values in every row."""
        seen = set()
        for slot, n_new in step:
            if not self.slots.is_held(slot):
                raise CacheError(f"slot {slot} is not open")
            if slot in seen:
                raise CacheError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            if n_new <= 0:
                raise CacheError(f"slot {slot}: a step brings {n_new} tokens")
            end = self.lengths[slot] + n_new
            if self.max_positions is not None and end > self.max_positions:
                raise CacheError(f"slot {slot}: position {end - 1} exceeds the model's {self.max_positions} positions")
            if end > self.max_blocks * PAGE:
                raise CacheError(f"slot {slot}: {end} positions exceed the cache's {self.max_blocks * PAGE} per sequence")
        for g in self.groups:
            missing = sum(g.pages_missing(slot, self.lengths[slot], n) for slot, n in step)
            if missing > g.pages.free:
                raise CacheError(f"the cache is full: this step needs {missing} more pages of {PAGE} positions, "
                                 f"{g.pages.free} of {g.pages.size} are free (max_tokens = {self.max_tokens})")
        tails = []
        for g in self.groups:
            of_group = []
            for slot, n in step:
                fresh = g.ensure(slot, self.lengths[slot], n)
                end = self.lengths[slot] + n
                last = (end - 1) // PAGE
                of_group.append((g.held[slot][last], end % PAGE) if last in fresh and end % PAGE else (-1, 0))
            tails.append(of_group)
        return tails

    def commit(self, step: list[tuple[int, int]]) -> None:
        """The step ran: lengths advance, window groups give back what fell out of the window."""
        for slot, n in step:
            self.lengths[slot] += n
            for g in self.groups:
                if g.need.kind == "window":
                    g.trim(slot, self.lengths[slot])

    def truncate(self, slot: int, length: int) -> None:
        """Forget the positions from `length` on (ember.cpp's `truncate`, graph_ir.cpp:3128).  Not
        possible where a window group has already given back pages that the shorter sequence
        would read, or where a layer keeps state that cannot drop tokens."""
        cur = self.length(slot)
        if not 0 <= length <= cur:
            raise CacheError(f"slot {slot}: cannot truncate {cur} positions to {length}")
        if any(s is not None for s in self.states) and length != cur:
            raise CacheError("a layer keeps per-sequence state; truncation would need a snapshot")
        for g in self.groups:
            first = g.first_needed_block(length)
            if any(p < 0 for p in g.held[slot][first:-(-length // PAGE)]):
                raise CacheError(f"slot {slot}: the window's pages before position {length} were given back")
        for g in self.groups:
            g.trim(slot, length)
        self.lengths[slot] = length

    def check(self) -> None:
        """Invariants: no slot or page lost, held twice or free while held."""
        self.slots.check()
        for g in self.groups:
            g.pages.check()
            owned = [p for s in range(self.n_slots) for p in g.held[s] if p >= 0]
            if len(owned) != len(set(owned)):
                raise PoolError("a page is held by two sequences")
            if len(owned) != g.pages.held:
                raise PoolError(f"pages lost: sequences hold {len(owned)}, the pool says {g.pages.held}")
            for s in range(self.n_slots):
                if g.held[s] and not self.slots.is_held(s):
                    raise PoolError(f"closed slot {s} still holds pages")
