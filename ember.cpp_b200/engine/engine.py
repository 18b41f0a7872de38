"""The step function: a batch of sequences, their new tokens in, the logits at the wanted places
out, the cache advanced.

ember.cpp's interpreter has `forward(tokens, start_pos, all_rows, tail_rows)` for one sequence:
the tokens sit at absolute positions start_pos.., the state must hold the positions before them,
and it returns the last row, every row or the last rows (graph_ir.h:115-124).  Its llama path runs a
batch's prompts concatenated in one call and then one token per active sequence per call
(api.cpp:1933-2063, 2212-2303).  All checks that a launch cannot make are made on the host first
(graph_ir.cpp:3733-3743, 3756-3758, 3897-3899), and an error leaves the state as it was
(tools/ir_adapter.cpp:244-245).  `Engine.step` is that for a batch of slots.
"""
from __future__ import annotations

import dataclasses

import numpy as np
import torch

from ..cache.sequence_cache import CacheError, SequenceCache
from ..config.base import ModelConfig, get_architecture, load_config
from ..options import RuntimeOptions
from ..parts.model import DecoderModel
from ..parts.spec import ModelSpec
from ..weights.loader import check_tensors, load_checked
from .plan import StepPlan, build_step

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


class StepError(ValueError):
    """A step that was refused on the host; nothing was launched and nothing changed."""


class Runtime:
    """Compute type, device and the kernels; prepares stored tensors for them."""

    def __init__(self, dtype, device, ops):
        self.dtype = DTYPES[dtype] if isinstance(dtype, str) else dtype
        if self.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute type {dtype!r} is not bfloat16 or float32")
        self.device = torch.device(device)
        self.ops = ops

    def matrix(self, t: torch.Tensor, transpose: bool = False) -> torch.Tensor:
        """[out, in] row-major in the compute type.  float32 compute widens bfloat16 exactly;
        bfloat16 compute rounds a matrix that was stored in 32-bit, which is what asking for
        bfloat16 means for a 32-bit checkpoint."""
        t = t.to(self.device)
        if transpose:
            t = t.t()
        return t.to(self.dtype).contiguous()

    def table(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(self.device).to(self.dtype).contiguous()

    def vector(self, t: torch.Tensor) -> torch.Tensor:
        """Biases and norm parameters are read as float32 by every kernel."""
        return t.to(self.device).to(torch.float32).contiguous()


@dataclasses.dataclass
class AppHandle:
    """What a mixer gets for one entry of the schedule."""
    index: int
    layer: int
    cache: object            # CacheView or None
    writes_cache: bool
    state: object            # tensor [slots, *shape] or None


@dataclasses.dataclass
class StepContext:
    ops: object
    dtype: torch.dtype
    plan: StepPlan
    apps: list
    position: object
    next_weights: tuple = ()   # set by the model: the first matrix that the block after the current one streams


class Engine:
    """A model, its cache and the step function."""

    def __init__(self, model: DecoderModel, runtime: Runtime, max_tokens: int, max_slots: int | None = None,
                 config: ModelConfig | None = None, cuda_graphs: bool = True, prompt_graphs: int = 0):
        self.model, self.runtime, self.config = model, runtime, config
        self.ops = runtime.ops
        spec = model.spec
        self.vocab_size = spec.vocab_size
        self.cache = SequenceCache(model.application_needs(), [a.cache_of for a in spec.schedule], max_tokens,
                                   model.max_positions(), runtime.dtype, runtime.device, max_slots)
        self.apps = [AppHandle(i, a.layer, self.cache.views[i], self.cache.writes[i], self.cache.states[i])
                     for i, a in enumerate(spec.schedule)]
        self._device_buffer = None
        self._staging = _Staging(runtime.device)
        self._graphs: dict[int, "_DecodeGraph"] = {}
        # Steps that bring prompts: a step whose shape (tokens, sequences, wanted rows, longest prompt and context)
        # has been seen before is captured as a graph too and replayed from then on, the last few shapes being kept
        # (`prompt_graphs` of them; 0: never).  Between the launches of a graph the device loses about a
        # microsecond less than between launches from the host, some 500 times in a step of a large model.
        self.prompt_graphs = int(prompt_graphs)
        self._prompt_graphs: dict[tuple, "_DecodeGraph"] = {}
        self._prompt_seen: dict[tuple, int] = {}
        # Where a sampler leaves a step's ids for the next step (`sample_target`): two halves in turn, at an
        # address that a captured step can name.  The step that reads one half is queued before the sampler
        # that writes the other, and the host has read a half's ids before the half is written again.
        self._ids_ring = None
        self._ids_turn = 0
        # a part whose forward does work on the host (reads a value back, loops over tokens in
        # Python) cannot be replayed from a captured graph; it says so with graph_safe = False
        # (per-launch timing needs an event between launches, which a captured graph does not carry)
        self.cuda_graphs = (bool(cuda_graphs) and runtime.device.type == "cuda"
                            and not getattr(self.ops, "op_timing", False)
                            and all(getattr(p, "graph_safe", True) for p in model.all_parts()))
        self.counters = {"steps": 0, "prompt_tokens": 0, "decode_tokens": 0}

    # ------------------------------------------------------------------ construction
    @staticmethod
    def _options(options, dtype, max_tokens, max_slots, cuda_graphs) -> RuntimeOptions:
        """The options an engine runs with: `options` (default: the defaults with the EMBER_*
        variables laid on top), with the arguments that were given in their own right on top."""
        base = options if options is not None else RuntimeOptions.from_env()
        return base.replace(dtype=dtype, max_tokens=max_tokens, max_slots=max_slots, cuda_graphs=cuda_graphs)

    @classmethod
    def from_folder(cls, folder: str, dtype=None, max_tokens: int | None = None, device="cuda", ops=None,
                    max_slots: int | None = None, cuda_graphs: bool | None = None,
                    options: RuntimeOptions | None = None) -> "Engine":
        """Config, model class and weights from `<folder>/config.json` and `model.safetensors`.
        `options`: a RuntimeOptions (compute type, cache size, kernel switches); dtype, max_tokens,
        max_slots and cuda_graphs given here override its fields."""
        opt = cls._options(options, dtype, max_tokens, max_slots, cuda_graphs)
        config = load_config(folder)
        config.check_dtype(opt.dtype)
        spec = get_architecture(config.architecture).build_spec(config)
        model = DecoderModel(spec)
        runtime = Runtime(opt.dtype, device, ops if ops is not None else _cuda_ops(opt))
        tensors = load_checked(folder, model.weight_specs(), spec.ignored_tensors, spec.strip_prefixes)
        model.load(tensors, runtime)
        return cls(model, runtime, opt.max_tokens, opt.max_slots, config, opt.cuda_graphs, opt.prompt_graphs)

    @classmethod
    def from_spec(cls, spec: ModelSpec, tensors: dict, dtype=None, max_tokens: int | None = None, device="cuda",
                  ops=None, max_slots: int | None = None, cuda_graphs: bool | None = None,
                  options: RuntimeOptions | None = None) -> "Engine":
        """A model given as data, with its tensors by name (how tests build toy models)."""
        opt = cls._options(options, dtype, max_tokens, max_slots, cuda_graphs)
        model = DecoderModel(spec)
        runtime = Runtime(opt.dtype, device, ops if ops is not None else _cuda_ops(opt))
        model.load(check_tensors("tensors", tensors, model.weight_specs(), spec.ignored_tensors, spec.strip_prefixes), runtime)
        return cls(model, runtime, opt.max_tokens, opt.max_slots, None, opt.cuda_graphs, opt.prompt_graphs)

    # ------------------------------------------------------------------ sequences
    def open(self) -> int:
        return self.cache.open()

    def close(self, slot: int) -> None:
        self.cache.close(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ------------------------------------------------------------------ the step
    def check_step(self, entries) -> None:
        if not entries:
            raise StepError("a step without sequences")
        for slot, tokens, want in entries:
            if len(tokens) == 0:
                raise StepError(f"slot {slot}: a step brings no tokens")
            bad = [int(t) for t in tokens if not 0 <= int(t) < self.vocab_size]
            if bad:
                raise StepError(f"slot {slot}: token id {bad[0]} is outside the vocabulary [0, {self.vocab_size})")
            for w in want:
                if not 0 <= int(w) < len(tokens):
                    raise StepError(f"slot {slot}: wanted place {w} is not among its {len(tokens)} new tokens")

    def prepare(self, entries, pad_to: int = 0, want_all: bool = False, device_tokens=None):
        """Checks a step, takes its pages and builds its description; launches nothing."""
        self.check_step(entries)
        rows = None
        if device_tokens is not None:
            ids, rows = device_tokens
            rows = [int(r) for r in rows]
            if len(rows) != len(entries) or any(len(t) != 1 for _, t, _ in entries):
                raise StepError("tokens taken from the device: one row for each sequence, one token a sequence")
            if ids.dtype != torch.int32 or ids.dim() != 1 or any(not 0 <= r < ids.shape[0] for r in rows):
                raise StepError("tokens taken from the device: rows of a one-dimensional int32 tensor of sampled ids")
        shape = [(slot, len(tokens)) for slot, tokens, _ in entries]
        try:
            tails = self.cache.reserve(shape)
        except CacheError as e:
            raise StepError(str(e)) from None
        tables = [g.table for g in self.cache.groups]
        return build_step(entries, self.cache.lengths, tables, self.cache.max_blocks, pad_to, want_all, rows, tails), shape

    def clear_tails(self, plan: StepPlan) -> None:
        """Clears the rows past the step's end in pages that are new to their sequences (see
        `SequenceCache.reserve`), in every layer's keys and values.  Before the step's own launches,
        and outside a captured graph: most steps have none."""
        if not plan.has_tails:
            return
        for g, group in enumerate(self.cache.groups):
            self.ops.clear_tails(group, plan.tails[g])

    def _stage(self, staging: "_Staging", host, device_buffer) -> None:
        """Host description -> pinned memory -> device, without racing an earlier copy."""
        n = host.packed.shape[0]
        staging.write(host.packed)
        device_buffer[:n].copy_(staging.pinned[:n], non_blocking=True)
        staging.copied()

    def upload(self, host) -> StepPlan:
        n = host.packed.shape[0]
        if self._device_buffer is None or self._device_buffer.numel() < n:
            self._device_buffer = torch.empty(max(n, 4096), dtype=torch.int32, device=self.runtime.device)
        self._stage(self._staging, host, self._device_buffer)
        return StepPlan(host, self._device_buffer)

    def step(self, entries, borrow: bool = False, device_tokens=None) -> torch.Tensor | None:
        """entries: (slot, tokens, want) per sequence; `want` lists the places among this step's
        tokens whose logits are returned.  Returns float32 [sum of wants, vocab] on the device,
        in the order of the entries and of `want` (None if nothing is wanted).  With `borrow` the
        result may be a view of a buffer that the next step overwrites.
        device_tokens = (ids, rows): every sequence brings one token, and the token of entry i is
        ids[rows[i]], an id that an earlier step's sampler left on the device (the entry's own
        token value is a placeholder).  The step can then be queued before the host has read
        those ids."""
        if self.cuda_graphs and all(len(t) == 1 for _, t, _ in entries):
            return self._graph_step(entries, borrow, device_tokens)
        host, shape = self.prepare(entries, device_tokens=device_tokens)
        g = self._prompt_graph(host) if device_tokens is None else None
        if g is not None:
            g.replay(self, host)
            self._account(host, shape)
            return g.logits if g.logits is None or borrow else g.logits.clone()
        plan = self.upload(host)
        if device_tokens is not None:
            self.ops.take_tokens(plan.tokens, plan.token_src, device_tokens[0], self.vocab_size)
        self.clear_tails(plan)
        logits = self.run(plan)
        self._account(host, shape)
        return logits

    PROMPT_GRAPH_TOKENS = 8192   # a captured step keeps its activations' memory: larger steps are launched from the host

    def _prompt_graph(self, host):
        """The captured graph of a step of this shape, made when the shape comes for the second time; None for
        a shape that is new (it runs launch by launch) or when such graphs are off."""
        if not (self.prompt_graphs > 0 and self.cuda_graphs) or host.T > self.PROMPT_GRAPH_TOKENS:
            return None
        key = (host.T, host.n, host.n_want, host.max_new, -(-host.max_end // 64), host.all_from_zero,
               host.wants_every_row, host.packed.shape[0])
        g = self._prompt_graphs.pop(key, None)
        if g is None:
            if len(self._prompt_seen) > 4096:
                self._prompt_seen.clear()
            self._prompt_seen[key] = self._prompt_seen.get(key, 0) + 1
            if self._prompt_seen[key] < 2:
                return None
            while len(self._prompt_graphs) >= self.prompt_graphs:       # the shape used longest ago goes
                self._prompt_graphs.pop(next(iter(self._prompt_graphs)))
            g = _DecodeGraph(self, host, None)
        self._prompt_graphs[key] = g                                    # (most recently used last)
        return g

    def _account(self, host, shape) -> None:
        self.cache.commit(shape)
        self.counters["steps"] += 1
        self.counters["decode_tokens" if host.all_single else "prompt_tokens"] += sum(n for _, n in shape)

    def run(self, plan: StepPlan):
        ctx = StepContext(self.ops, self.runtime.dtype, plan, self.apps, self.model.position)
        if getattr(self.ops, "nvtx", False):
            torch.cuda.nvtx.range_push(f"step {'decode' if plan.all_single else 'prefill'} T={plan.T} n={plan.n}")
            try:
                return self.model.forward(ctx)
            finally:
                torch.cuda.nvtx.range_pop()
        return self.model.forward(ctx)

    def sample_target(self, rows: int):
        """An int32 tensor of `rows` entries for a sampler to write a step's ids into, from which the next
        step can take its tokens without a launch of its own (`step(device_tokens=(that tensor, rows))`)."""
        ring, cap = self._ring(), max(self.cache.n_slots, 1)
        if rows > cap:
            raise StepError(f"{rows} rows of sampled ids, but the cache has {cap} slots")
        self._ids_turn ^= 1
        return ring[self._ids_turn * cap: self._ids_turn * cap + rows]

    def _ring(self):
        if self._ids_ring is None:
            self._ids_ring = torch.zeros(2 * max(self.cache.n_slots, 1), dtype=torch.int32, device=self.runtime.device)
        return self._ids_ring

    def _ring_rows(self, ids, rows):
        """`rows` of `ids` as rows of the ring that captured steps read: `ids` is a piece of the ring (what
        `sample_target` gave out), or is copied into the ring's next piece first."""
        ring = self._ring()
        if (not torch.is_tensor(ids) or ids.dtype != torch.int32 or ids.dim() != 1 or ids.device != ring.device
                or not ids.is_contiguous() or any(not 0 <= int(r) < ids.shape[0] for r in rows)):
            raise StepError("tokens taken from the device: rows of a one-dimensional int32 tensor of sampled ids")
        off = ids.data_ptr() - ring.data_ptr()
        if not (off >= 0 and off % 4 == 0 and off // 4 + ids.shape[0] <= ring.numel()):
            if ids.shape[0] > max(self.cache.n_slots, 1):
                raise StepError(f"tokens taken from the device: {ids.shape[0]} sampled ids, but the cache has "
                                f"{self.cache.n_slots} slots")
            piece = self.sample_target(ids.shape[0])
            piece.copy_(ids)
            off = piece.data_ptr() - ring.data_ptr()
        return ring, [off // 4 + int(r) for r in rows]

    # ------------------------------------------------------------------ one token each, as a replayed graph
    def _length_bucket(self, pages: int) -> int:
        """The pages of the longest sequence, rounded up to 4, 6, 8, 12, 16, 24, ... (or to all the cache
        gives a sequence): a captured graph's launches are sized for that many, so that the attention
        can cut a short context and a long one differently."""
        top = self.cache.max_blocks
        size = 4
        while size < pages and size < top:
            size = size * 3 // 2 if (size & (size - 1)) == 0 else size * 4 // 3
        return min(size, top)

    def capture_decode(self, batch: int) -> int:
        """Captures the one-token step's graphs for batches of up to `batch` sequences (its bucket) at every
        bucket of lengths, with padding in place of sequences, so that no later step pays for a capture.
        Returns how many graphs were captured."""
        bucket = 1
        while bucket < batch:
            bucket *= 2
        made, pages = 0, 0
        while pages < self.cache.max_blocks:
            pages = self._length_bucket(pages + 1)
            if (bucket, pages) not in self._graphs:
                tables = [g.table for g in self.cache.groups]
                host = build_step([], self.cache.lengths, tables, self.cache.max_blocks, bucket, True, None)
                self._graphs[(bucket, pages)] = _DecodeGraph(self, host, pages)
                made += 1
        return made

    def _graph_step(self, entries, borrow: bool, device_tokens=None):
        """A step in which every sequence brings one token runs as a CUDA graph captured once per
        bucket of batch sizes and of lengths (ember.cpp captures its one-token step once and replays
        it with [token, pos, kv_row] in device memory, graph_ir.cpp:4306-4373).  The batch is padded
        to the bucket with sequences of slot -1; the description of the step is the only thing that
        changes between replays."""
        n_real = len(entries)
        bucket = 1
        while bucket < n_real:
            bucket *= 2
        if device_tokens is not None:     # the captured step's embedding takes them from the ring itself
            device_tokens = self._ring_rows(*device_tokens)
        host, shape = self.prepare(entries, pad_to=bucket, want_all=True, device_tokens=device_tokens)
        pages = self._length_bucket(-(-host.max_end // 64))
        g = self._graphs.get((bucket, pages))
        if g is None:
            g = self._graphs[(bucket, pages)] = _DecodeGraph(self, host, pages)
        g.replay(self, host)
        self._account(host, shape)
        rows = [i for i, (_, _, want) in enumerate(entries) for _ in want]
        if not rows:
            return None
        if rows == list(range(n_real)):
            out = g.logits[:n_real]
        else:
            out = g.logits[torch.tensor(rows, device=g.logits.device)]
            borrow = True
        return out if borrow else out.clone()


class _Staging:
    """A pinned host buffer that is not rewritten before its last copy to the device has run."""

    def __init__(self, device):
        self.cuda = torch.device(device).type == "cuda"
        self.pinned = None
        self.event = None

    def write(self, packed: np.ndarray) -> None:
        n = packed.shape[0]
        if self.event is not None:
            self.event.synchronize()
        if self.pinned is None or self.pinned.numel() < n:
            self.pinned = torch.empty(max(n, 4096), dtype=torch.int32, pin_memory=self.cuda)
        self.pinned[:n].numpy()[:] = packed

    def copied(self) -> None:
        if self.cuda:
            if self.event is None:
                self.event = torch.cuda.Event()
            self.event.record()


class _DecodeGraph:
    """A step captured once and replayed with a new description in its buffer: the one-token step of a bucket of
    batch sizes and lengths (`pages`: the pages its launches are sized for), or a step of prompts of one shape
    (`pages` None: sized as the step is)."""

    def __init__(self, engine: Engine, host, pages: int | None):
        dev = engine.runtime.device
        self.buffer = torch.zeros(host.packed.shape[0], dtype=torch.int32, device=dev)
        self.staging = _Staging(dev)
        self.size = host.packed.shape[0]
        # launches are sized for sequences of up to `pages` pages, lengths come from the buffer
        sized = host if pages is None else dataclasses.replace(host, max_end=pages * 64)
        self.plan = StepPlan(sized, self.buffer)
        if dev.type == "cuda":            # tokens that an earlier step's sampler left in the ring are taken by the embedding
            self.plan.device_ids = engine._ring()
        engine._stage(self.staging, host, self.buffer)
        engine.clear_tails(self.plan)
        if dev.type != "cuda":
            self.graph = None
            return
        # once without capture: libraries choose their algorithms and allocate outside the graph
        engine.run(self.plan)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        before = engine.ops.launches
        with torch.cuda.graph(self.graph):
            self.logits = engine.run(self.plan)
        self.launches = engine.ops.launches - before

    def replay(self, engine: Engine, host) -> None:
        if host.packed.shape[0] != self.size:
            raise StepError("the step's description changed size under a captured graph")
        engine._stage(self.staging, host, self.buffer)
        if host.has_tails:            # outside the graph as well: a step in 64 has any
            self.plan.has_tails = True
            engine.clear_tails(self.plan)
        if self.graph is None:
            self.logits = engine.run(self.plan)
        else:
            self.graph.replay()
            engine.ops.launches += self.launches


def _cuda_ops(options=None):
    from ..csrc.ops import CudaOps
    return CudaOps(options)
