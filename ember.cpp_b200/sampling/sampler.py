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


class Sampler:
    """Draws one token per row of logits on the device."""

    def __init__(self, ops):
        self.ops = ops

    def sample(self, logits: torch.Tensor, params: SamplingParams, streams, counters) -> torch.Tensor:
        """logits: float32 [rows, vocab] on the device.  streams, counters: one int per row (lists
        or int32 tensors).  Returns int32 [rows] on the device."""
        dev = logits.device
        if not torch.is_tensor(streams):
            streams = torch.tensor(list(streams), dtype=torch.int32, device=dev)
        if not torch.is_tensor(counters):
            counters = torch.tensor(list(counters), dtype=torch.int32, device=dev)
        return self.ops.sample(logits, params.temperature, params.top_k, params.top_p, params.seed, streams, counters)
