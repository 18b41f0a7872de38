"""The generation loop above the step function.

ember.cpp's `generate` runs the prompt in one call, samples, then one token per call until a stop
id, `steps` new tokens or the end of the context (api.cpp:989-991, 1071-1091, 1166-1174,
1355-1356, 1512-1521); its `generate_batch` does the same for a batch: all prompts in one call,
then per step the sequences that are still active, each leaving when it has sampled its stop id,
until all are finished or `steps` is reached (api.cpp:1646-1891).  Here: requests are cut into
batches that fit the batch size and the cache, each batch's prompts run in one step, then one
token each; a sequence that ends gives its slot back at once; batches follow one another until
every request is served.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Sequence

from ..cache.sequence_cache import PAGE
from ..sampling.sampler import Sampler, SamplingParams


@dataclasses.dataclass(frozen=True)
class GenerationParams:
    max_new_tokens: int = 128            # ember.cpp's `steps`
    sampling: SamplingParams = SamplingParams()
    stop_token_ids: tuple[int, ...] | None = None   # None: the model's own (its eos id, if it has one)
    max_batch_size: int = 8              # ember.cpp's --max-batch-size default (main.cpp:128)


@dataclasses.dataclass
class Generation:
    tokens: list[int]
    finish_reason: str                   # "stop" | "length" | "context"


class GenerationError(ValueError):
    pass


def finish_reason(token: int, n_generated: int, n_cached: int, stop_ids, max_new_tokens: int,
                  max_positions: int | None) -> str | None:
    """Decides, after `token` was sampled, whether the sequence ends.  `n_cached` positions are in
    the cache (the sampled token is not yet among them).  Order as in ember.cpp: the stop id
    first (api.cpp:1512-1516), then the count of new tokens (:1518-1521), then the context
    (:1169-1174)."""
    if token in stop_ids:
        return "stop"
    if n_generated >= max_new_tokens:
        return "length"
    if max_positions is not None and n_cached + 1 > max_positions:
        return "context"
    return None


def plan_batches(prompt_lengths: Sequence[int], max_new_tokens: int, max_batch_size: int, max_tokens: int,
                 max_positions: int | None, max_slots: int | None = None) -> list[list[int]]:
    """Cuts the requests, in order, into batches.  A batch holds at most `max_batch_size` requests
    (and slots), and the pages its sequences can come to hold (prompt plus new tokens, bounded by
    the context, rounded up to whole pages) fit `max_tokens`."""
    if max_batch_size <= 0:
        raise GenerationError(f"max_batch_size = {max_batch_size} must be positive")
    limit = max_batch_size if max_slots is None else min(max_batch_size, max_slots)
    batches: list[list[int]] = []
    current: list[int] = []
    used = 0
    for i, n in enumerate(prompt_lengths):
        if n <= 0:
            raise GenerationError(f"request {i} has an empty prompt")
        if max_positions is not None and n > max_positions:
            raise GenerationError(f"request {i}: its prompt of {n} tokens exceeds the model's {max_positions} positions")
        # the last sampled token is never fed, so a sequence holds at most n + max_new_tokens - 1 positions
        most = n + max(max_new_tokens - 1, 0)
        if max_positions is not None:
            most = min(most, max_positions)
        need = -(-most // PAGE) * PAGE
        if need > max_tokens:
            raise GenerationError(f"request {i} can come to hold {need} cache positions, the cache has {max_tokens}")
        if current and (len(current) >= limit or used + need > max_tokens):
            batches.append(current)
            current, used = [], 0
        current.append(i)
        used += need
    if current:
        batches.append(current)
    return batches


class Generator:
    def __init__(self, engine, sampler: Sampler | None = None, run_ahead: bool = True):
        self.engine = engine
        self.sampler = sampler or Sampler(engine.ops)
        self.run_ahead = bool(run_ahead) and hasattr(engine.ops, "take_tokens")
        self.stats = {"batches": 0, "prefill_steps": 0, "decode_steps": 0, "prompt_tokens": 0, "new_tokens": 0}

    def generate(self, prompts: Sequence[Sequence[int]], params: GenerationParams = GenerationParams(),
                 on_token: Callable[[int, int], None] | None = None, first_stream: int = 0) -> list[Generation]:
        """prompts: token ids per request.  Returns one Generation per request, in order.
        `on_token(request index, token)` is called for every new token as it is sampled (ember.cpp's
        token callback, api.h:243).  `first_stream` numbers the first request for the sampler."""
        eng = self.engine
        if params.max_new_tokens <= 0:
            raise GenerationError(f"max_new_tokens = {params.max_new_tokens} must be positive")
        stop_ids = params.stop_token_ids if params.stop_token_ids is not None else eng.model.spec.stop_token_ids
        stop_ids = frozenset(int(t) for t in stop_ids)
        max_pos = eng.model.max_positions()
        batches = plan_batches([len(p) for p in prompts], params.max_new_tokens, params.max_batch_size,
                               eng.cache.max_tokens, max_pos, eng.cache.n_slots)
        results: list[Generation | None] = [None] * len(prompts)
        for batch in batches:
            self._run_batch(batch, prompts, params, stop_ids, max_pos, results, on_token, first_stream)
        return results  # type: ignore[return-value]

    def _run_batch(self, batch, prompts, params, stop_ids, max_pos, results, on_token, first_stream) -> None:
        """One batch from its prompts to its last token.

        The loop runs one step ahead of what the host has read: a step's tokens stay on the device
        and the next step takes them from there (`Engine.step(device_tokens=...)`), so the host
        queues step t+1, then reads step t's ids (by then long computed) and decides who ended.
        Whether a sequence ends by its count of new tokens or by the context is known without the
        token; a stop id is not, so a sequence that drew one has been stepped once more for
        nothing: that row is dropped, and its slot is closed like any other."""
        eng = self.engine
        self.stats["batches"] += 1
        slots = {i: eng.open() for i in batch}
        generated: dict[int, list[int]] = {i: [] for i in batch}

        def launch(active, entries, device_tokens):
            logits = eng.step(entries, borrow=device_tokens is not None, device_tokens=device_tokens)
            target = getattr(eng, "sample_target", None)   # where the next step can take the ids from by itself
            ids = self.sampler.sample(logits, params.sampling, [first_stream + i for i in active],
                                      [len(generated[i]) + (device_tokens is not None) for i in active],
                                      out=None if target is None or not logits.is_cuda else target(len(active)))
            # (requests, their ids on the device and on the way to the host, positions in the cache after the step)
            return active, ids, self.sampler.fetch(ids), [eng.length(slots[i]) for i in active]

        try:
            active = list(batch)
            self.stats["prefill_steps"] += 1
            self.stats["prompt_tokens"] += sum(len(prompts[i]) for i in active)
            pending = launch(active, [(slots[i], list(prompts[i]), [len(prompts[i]) - 1]) for i in active], None)
            while pending is not None:
                active, ids, on_the_way, cached = pending
                following = None
                if self.run_ahead:
                    # who goes on whatever token was drawn: not those at their count or at the context's end
                    ahead = [(row, i) for row, i in enumerate(active)
                             if results[i] is None and len(generated[i]) + 1 < params.max_new_tokens
                             and not (max_pos is not None and cached[row] + 1 > max_pos)]
                    if ahead:
                        self.stats["decode_steps"] += 1
                        following = launch([i for _, i in ahead], [(slots[i], [0], [0]) for _, i in ahead],
                                           (ids, [row for row, _ in ahead]))
                tokens = on_the_way.tolist()   # waits for the step that drew them; the next one is queued already
                for row, (i, tok) in enumerate(zip(active, tokens)):
                    if results[i] is not None:
                        continue           # it ended a step ago on a stop id: this row was computed for nothing
                    generated[i].append(tok)
                    self.stats["new_tokens"] += 1
                    if on_token is not None:
                        on_token(i, tok)
                    why = finish_reason(tok, len(generated[i]), cached[row], stop_ids, params.max_new_tokens, max_pos)
                    if why is not None:
                        results[i] = Generation(generated[i], why)
                        eng.close(slots.pop(i))   # the slot and its pages are free for the next batch at once
                if following is None and not self.run_ahead:
                    still = [i for i in active if results[i] is None]
                    if still:
                        self.stats["decode_steps"] += 1
                        pending = launch(still, [(slots[i], [generated[i][-1]], [0]) for i in still], None)
                        continue
                pending = following
            check = getattr(eng.ops, "check", None)
            if check is not None:
                check()        # a kernel whose bounded wait ran out has said so (every id has been read: the device is idle)
        finally:
            for slot in slots.values():
                eng.close(slot)
