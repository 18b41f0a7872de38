"""Interfaces of the parts and their registry.

A part is built from a `PartSpec` alone: its sizes and constants are constructor parameters, its
tensors are named by a prefix that the architecture gives it.  No part knows which model it is in.

Roles and what each must provide:

  norm      forward(ctx, x, out_dtype) -> tensor                     (x: fp32 residual stream)
  mixer     forward(ctx, h, residual, app) -> new residual stream    (h: normed input)
            cache_need() -> CacheNeed | None, state_need() -> StateNeed | {name: StateNeed} | None
  ffn       forward(ctx, h, residual) -> new residual stream
  position  embedding_table() -> tensor | None, max_positions() -> int | None,
            apply_qk(ctx, qkv, n_heads, kv_heads, head_dim) (in place; default: nothing)
  block     forward(ctx, x, app) -> x       (the arrangement of the four parts above)

Every part lists its tensors with `weight_specs()` (name, stored shape, how random-weights mode
fills it) and receives them in `load(get, runtime)`.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable

from .spec import PartSpec


@dataclasses.dataclass(frozen=True)
class WeightSpec:
    """One tensor of a checkpoint: its full name, its shape as stored, and how the
    random-weights mode draws it: N(mean, std)."""
    name: str
    shape: tuple[int, ...]
    mean: float = 0.0
    std: float = 0.02
    integer: bool = False     # an integer table (kept as int32); none in GPT-2


@dataclasses.dataclass(frozen=True)
class CacheNeed:
    """What a mixer wants from the cache: all keys (`full`) or the last `window` of them."""
    kind: str                 # "full" | "window"
    kv_heads: int
    head_dim: int
    window: int = 0


@dataclasses.dataclass(frozen=True)
class StateNeed:
    """Per-sequence state of fixed size: `shape` values of `dtype` ("float32" or "int32") per
    sequence, set to `init` when a sequence starts.  A mixer that keeps several tensors returns a
    dict of these by name from `state_need()`, and finds a dict of tensors in `app.state`."""
    shape: tuple[int, ...]
    init: float = 0.0
    dtype: str = "float32"


class Part:
    role = ""
    # False for a part whose forward works on the host (reads device values back, loops in Python):
    # an engine with such a part runs every step launch by launch instead of replaying a graph
    graph_safe = True

    def __init__(self, prefix: str = ""):
        self.prefix = prefix

    def weight_specs(self) -> list[WeightSpec]:
        return []

    def stream_weights(self) -> list:
        """The weight matrices that this part's forward streams through `ops.linear`, in that order
        (as prepared by load()).  A hint for the kernels: a block announces them so that one product's
        launch can ask the next product's weights into L2.  The default names none."""
        return []

    def load(self, get: Callable[[str], Any], runtime) -> None:
        """Fetch the tensors named in weight_specs() with `get(name)` (as stored, on the
        runtime's device) and keep them in the form the kernels want."""


class Norm(Part):
    role = "norm"

    def forward(self, ctx, x, out_dtype):
        raise NotImplementedError


class Mixer(Part):
    role = "mixer"

    def cache_need(self) -> CacheNeed | None:
        return None

    def state_need(self) -> "StateNeed | dict[str, StateNeed] | None":
        return None

    def forward(self, ctx, h, residual, app):
        raise NotImplementedError


class FeedForward(Part):
    role = "ffn"

    def forward(self, ctx, h, residual):
        raise NotImplementedError


class Position(Part):
    role = "position"

    def embedding_table(self):
        return None

    def max_positions(self) -> int | None:
        return None

    def apply_qk(self, ctx, qkv, n_heads: int, kv_heads: int, head_dim: int) -> None:
        return None


class Block(Part):
    role = "block"

    def __init__(self, norm1: "Norm | None", mixer: Mixer, norm2: "Norm | None", ffn: FeedForward, **more_norms: Norm):
        super().__init__("")
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self.more_norms = dict(more_norms)     # the arrangement's further norms, by the names the spec gives them

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn, *self.more_norms.values()) if p is not None]

    def forward(self, ctx, x, app):
        raise NotImplementedError


_REGISTRY: dict[str, dict[str, Callable[..., Part]]] = {r: {} for r in ("norm", "mixer", "ffn", "position", "block")}


def register_part(role: str, kind: str, factory: Callable[..., Part]) -> None:
    """Makes `kind` available to specs for `role`.  `factory(prefix=..., **params)` builds the
    part (for a block: `factory(norm1, mixer, norm2, ffn, **more_norms)`; a norm the spec leaves
    out arrives as None)."""
    if role not in _REGISTRY:
        raise ValueError(f"unknown role {role!r}; roles: {sorted(_REGISTRY)}")
    _REGISTRY[role][kind] = factory


def registered(role: str) -> list[str]:
    return sorted(_REGISTRY[role])


def build_part(role: str, spec: PartSpec) -> Part:
    kinds = _REGISTRY[role]
    if spec.kind not in kinds:
        raise ValueError(f"no {role} of kind {spec.kind!r} is registered; registered: {registered(role)}")
    return kinds[spec.kind](prefix=spec.prefix, **spec.params)


def build_block(kind: str, norm1, mixer, norm2, ffn, more_norms=None) -> Block:
    kinds = _REGISTRY["block"]
    if kind not in kinds:
        raise ValueError(f"no block arrangement {kind!r} is registered; registered: {registered('block')}")
    return kinds[kind](norm1, mixer, norm2, ffn, **(more_norms or {}))
