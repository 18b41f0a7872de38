"""The description of one step that the kernels read: which tokens, at which positions, of which
sequences, in which pages.

ember.cpp's batch path gathers, per step, the active sequences' (token, position, original index)
(api.cpp:1819-1834) and gives prompt lengths beside the concatenated prompts
(api.cpp:1961-2011); its graph replay keeps [token, pos, kv_row] in device memory
(graph_ir.cpp:4361-4364).  Here a step is one packed int32 buffer, built on the host and copied
once:

  tokens[T] positions[T] token_seq[T]            one entry per token, sequences back to back
  token_src[T]                                   -1, or the row of an earlier step's sampled ids that is this token
  seq_slot[n] seq_start[n] seq_new[n] cu_new[n+1] one entry per sequence (slot -1: padding)
  want_rows[R]                                   rows of the token list whose logits are wanted
  pages[g][n, max_blocks]                        per cache group, each sequence's page numbers
  tails[g][n, 2]                                 per cache group and sequence: (page, first row) of a new page's
                                                 rows past the step's end, which are cleared first, or (-1, 0)

Padding sequences (slot -1, no tokens of their own in prefill; one dummy token in a padded decode
batch) are skipped by every kernel that touches the cache and change no result.
"""
from __future__ import annotations

import dataclasses

import numpy as np


@dataclasses.dataclass
class StepLayout:
    """Offsets (in int32 elements) of the fields inside the packed buffer."""
    T: int
    n: int
    R: int
    max_blocks: int
    n_groups: int

    def __post_init__(self):
        off = 0

        def take(count):
            nonlocal off
            start = off
            off += -(-count // 4) * 4  # fields start on 16-byte boundaries
            return start

        self.tokens = take(self.T)
        self.positions = take(self.T)
        self.token_seq = take(self.T)
        self.token_src = take(self.T)
        self.seq_slot = take(self.n)
        self.seq_start = take(self.n)
        self.seq_new = take(self.n)
        self.cu_new = take(self.n + 1)
        self.want_rows = take(max(self.R, 1))
        self.pages = [take(self.n * self.max_blocks) for _ in range(self.n_groups)]
        self.tails = [take(2 * self.n) for _ in range(self.n_groups)]
        self.size = off


@dataclasses.dataclass
class HostStep:
    """A checked step on the host: the packed buffer and the facts kernels are launched with."""
    layout: StepLayout
    packed: np.ndarray            # int32 [layout.size]
    T: int                        # tokens in the step (with padding tokens)
    n: int                        # sequences (with padding sequences)
    n_want: int
    max_new: int                  # most new tokens of one sequence
    max_end: int                  # longest sequence after the step
    all_from_zero: bool           # every real sequence starts at position 0
    all_single: bool              # every sequence brings one token
    wants_every_row: bool = False # the wanted rows are all rows, in order
    has_tails: bool = False       # some sequence's new last page has rows to clear before the step


def build_step(entries, lengths, page_tables, max_blocks: int, pad_to: int = 0, want_all: bool = False,
               token_rows=None, tails=None) -> HostStep:
    """entries: (slot, tokens, want) per sequence, `want` being indices into that sequence's new
    tokens.  lengths: slot -> positions held before the step.  page_tables: per group, a function
    (slots, width) -> int32 [n, width].  pad_to: pad a one-token-each batch with dummy sequences
    up to this many (0: no padding).  want_all: every token's row is wanted, padding included, and
    the entries' own `want` is left to the caller (the shape a replayed graph needs).  token_rows:
    per entry the row of a device array of sampled ids that holds its (single) token, which the
    device puts in place of the entry's own token value.  tails: what `SequenceCache.reserve`
    returned for this step (per group and entry, (page, first row) to clear, or (-1, 0))."""
    n_real = len(entries)
    single = all(len(t) == 1 for _, t, _ in entries)
    n = max(n_real, pad_to) if (single and pad_to) else n_real
    T = sum(len(t) for _, t, _ in entries) + (n - n_real)
    R = T if want_all else sum(len(w) for _, _, w in entries)
    lay = StepLayout(T, n, R, max_blocks, len(page_tables))
    buf = np.zeros(lay.size, dtype=np.int32)
    buf[lay.token_src:lay.token_src + T] = -1
    if token_rows is not None and (len(token_rows) != n_real or not single):
        raise ValueError("tokens taken from the device: one row for each entry, one token an entry")
    slots = []
    t0 = 0
    r0 = 0
    max_new = max_end = 0
    from_zero = True
    for i in range(n):
        if i < n_real:
            slot, toks, want = entries[i]
            start = lengths[slot]
        else:
            slot, toks, want, start = -1, [0], (), 0
        k = len(toks)
        slots.append(slot)
        buf[lay.tokens + t0: lay.tokens + t0 + k] = toks
        buf[lay.positions + t0: lay.positions + t0 + k] = np.arange(start, start + k)
        buf[lay.token_seq + t0: lay.token_seq + t0 + k] = i
        if token_rows is not None and i < n_real:
            buf[lay.token_src + t0] = token_rows[i]
        buf[lay.seq_slot + i] = slot
        buf[lay.seq_start + i] = start
        buf[lay.seq_new + i] = k
        buf[lay.cu_new + i] = t0
        for w in (range(k) if want_all else want):
            if not 0 <= w < k:
                raise ValueError(f"sequence {i}: wanted place {w} is not among its {k} new tokens")
            buf[lay.want_rows + r0] = t0 + w
            r0 += 1
        t0 += k
        if slot >= 0:
            max_new = max(max_new, k)
            max_end = max(max_end, start + k)
            from_zero = from_zero and start == 0
    buf[lay.cu_new + n] = t0
    for g, table in enumerate(page_tables):
        buf[lay.pages[g]: lay.pages[g] + n * max_blocks] = table(slots, max_blocks).reshape(-1)
    has_tails = False
    for g in range(len(page_tables)):
        pairs = np.full((n, 2), (-1, 0), dtype=np.int32)
        if tails is not None:
            for i, (page, row) in enumerate(tails[g]):
                pairs[i] = (page, row)
                has_tails = has_tails or page >= 0
        buf[lay.tails[g]: lay.tails[g] + 2 * n] = pairs.reshape(-1)
    every = R == T and bool((buf[lay.want_rows:lay.want_rows + R] == np.arange(T)).all())
    return HostStep(lay, buf, T, n, R, max_new, max_end, from_zero, single, every, has_tails)


class StepPlan:
    """The same step as the kernels see it: views into one device buffer."""

    def __init__(self, host: HostStep, device_buffer):
        lay = host.layout
        self.host = host
        self.buffer = device_buffer
        self.T, self.n, self.n_want = host.T, host.n, host.n_want
        self.max_new, self.max_end, self.max_blocks = host.max_new, host.max_end, lay.max_blocks
        self.all_from_zero, self.all_single = host.all_from_zero, host.all_single
        self.wants_every_row = host.wants_every_row

        def view(start, count):
            return device_buffer[start:start + count]

        self.tokens = view(lay.tokens, lay.T)
        self.positions = view(lay.positions, lay.T)
        self.token_seq = view(lay.token_seq, lay.T)
        self.token_src = view(lay.token_src, lay.T)
        self.seq_slot = view(lay.seq_slot, lay.n)
        self.seq_start = view(lay.seq_start, lay.n)
        self.seq_new = view(lay.seq_new, lay.n)
        self.cu_new = view(lay.cu_new, lay.n + 1)
        self.want_rows = view(lay.want_rows, max(lay.R, 1))
        self.pages = [view(p, lay.n * lay.max_blocks).view(lay.n, lay.max_blocks) for p in lay.pages]
        self.tails = [view(p, 2 * lay.n).view(lay.n, 2) for p in lay.tails]
        self.has_tails = host.has_tails
        self.device_ids = None   # set by the engine: the sampled ids that `token_src` indexes (a replayed step)
