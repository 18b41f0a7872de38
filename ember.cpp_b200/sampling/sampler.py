"""Sampling parameters with ember.cpp's names, meanings and defaults, and the device sampler.

ember.cpp's `sample_top_k_top_p_temperature(logits, temperature, top_k, top_p, rng)`
(api.cpp:238-341): a temperature below 0.05 means the first maximal index; `top_k` <= 0 or
>= vocabulary means no top-k; `top_p` >= 1 means no top-p; defaults temperature 0.1, top_k 40,
top_p 0.9 (main.cpp:134-136; bindings.cpp:172-184); the generator is seeded by `set_seed`
(api.h:240).  The kept set is ember.cpp's; the draw uses the counter-based uniform below, keyed by
(seed, stream, counter) = (seed, number of the request, number of the token), so a request's
tokens do not depend on what else is in its batch.
"""
from __future__ import annotations

import dataclasses

import torch

GREEDY_BELOW = 0.05  # api.cpp:246


@dataclasses.dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.1
    top_k: int = 40
    top_p: float = 0.9
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature = {self.temperature} is negative")
        if not self.top_p >= 0:
            raise ValueError(f"top_p = {self.top_p} is negative")

    @property
    def greedy(self) -> bool:
        return self.temperature < GREEDY_BELOW


def uniform01(seed: int, stream: int, counter: int) -> float:
    """The uniform number in [0, 1) of draw `counter` of request `stream`: a splitmix64 round over
    the three, top 24 bits.  The sampling kernel computes the same."""
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + stream * 0xBF58476D1CE4E5B9 + counter * 0x94D049BB133111EB
         + 0x2545F4914F6CDD1D) & mask
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & mask
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & mask
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


class IdsOnTheWay:
    """Sampled ids on their way to the host: the copy runs on a stream of its own as soon as the
    sampler has finished, beside whatever was queued on the main stream after it, so that reading
    the ids of one step does not wait for the step that was queued behind it."""

    def __init__(self, ids: torch.Tensor, stream, pinned):
        self.ids = ids                      # kept alive until the copy has run
        self.event = None
        self.host = None
        if ids.is_cuda:
            drawn = torch.cuda.Event()
            drawn.record()                  # on the stream the sampler ran on
            self.host = pinned[:ids.shape[0]]
            with torch.cuda.stream(stream):
                stream.wait_event(drawn)
                self.host.copy_(ids, non_blocking=True)
                self.event = torch.cuda.Event()
                self.event.record(stream)

    def tolist(self) -> list[int]:
        if self.event is None:
            return self.ids.tolist()
        self.event.synchronize()
        return self.host.tolist()


class Sampler:
    """Draws one token per row of logits on the device."""

    def __init__(self, ops):
        self.ops = ops
        self._stream = None
        self._pinned = []                   # four buffers in turn: a step's ids are read while later steps' are copied
        self._turn = 0
        self._hpinned = []                  # pinned staging for the per-row stream and counter numbers
        self._hturn = 0
        self._kept = None                   # (stream numbers, their device tensor, zeros of the same length)

    def fetch(self, ids: torch.Tensor) -> IdsOnTheWay:
        """Starts copying sampled ids to the host without stopping the stream they were drawn on."""
        if not ids.is_cuda:
            return IdsOnTheWay(ids, None, None)
        if self._stream is None:
            self._stream = torch.cuda.Stream(device=ids.device)
        n = ids.shape[0]
        self._turn = (self._turn + 1) % 4
        while len(self._pinned) < 4:
            self._pinned.append(torch.empty(max(n, 64), dtype=torch.int32, pin_memory=True))
        if self._pinned[self._turn].numel() < n:
            self._pinned[self._turn] = torch.empty(n, dtype=torch.int32, pin_memory=True)
        return IdsOnTheWay(ids, self._stream, self._pinned[self._turn])

    def sample(self, logits: torch.Tensor, params: SamplingParams, streams, counters, out=None) -> torch.Tensor:
        """logits: float32 [rows, vocab] on the device.  streams, counters: one int per row (lists
        or int32 tensors).  Returns int32 [rows] on the device (`out`, if one is given)."""
        more = {} if out is None else {"out": out}
        base = 0
        if not torch.is_tensor(streams) or not torch.is_tensor(counters):
            streams, counters = list(streams), list(counters)
            if counters and min(counters) == max(counters) and hasattr(self.ops, "sample_takes_base"):
                # the sequences of a batch start together, so one number counts for all rows: it goes as an
                # argument, and the stream numbers stay on the device from step to step (no copy a step)
                key = tuple(streams)
                if self._kept is None or self._kept[0] != key:
                    on_device, zeros = self._to_device(streams, [0] * len(streams), logits.device)
                    self._kept = (key, on_device, zeros)
                base, streams, counters = counters[0], self._kept[1], self._kept[2]
            else:
                streams, counters = self._to_device(streams, counters, logits.device)
        if base:
            more["counter_base"] = base
        return self.ops.sample(logits, params.temperature, params.top_k, params.top_p, params.seed, streams, counters, **more)

    def _to_device(self, streams: list[int], counters: list[int], dev):
        """Two lists of ints -> two int32 device tensors with one copy from pinned memory.  (A copy
        from ordinary host memory would first wait for everything queued on the stream, which is
        the step this sampler call is meant to be queued behind.)"""
        n = len(streams)
        both = torch.tensor(streams + counters, dtype=torch.int32)
        if dev.type != "cuda":
            return both[:n], both[n:]
        self._hturn = (self._hturn + 1) % 8
        while len(self._hpinned) < 8:
            self._hpinned.append([torch.empty(256, dtype=torch.int32, pin_memory=True), None])
        slot = self._hpinned[self._hturn]
        if slot[1] is not None:
            slot[1].synchronize()          # the copy that last read this buffer (eight calls ago) is over
        if slot[0].numel() < 2 * n:
            slot[0] = torch.empty(2 * n, dtype=torch.int32, pin_memory=True)
        slot[0][:2 * n] = both
        out = torch.empty(2 * n, dtype=torch.int32, device=dev)
        out.copy_(slot[0][:2 * n], non_blocking=True)
        slot[1] = torch.cuda.Event()
        slot[1].record()
        return out[:n], out[n:]
