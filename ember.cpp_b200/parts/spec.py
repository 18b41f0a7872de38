"""A model as data: which parts make up each layer, and in which order the layers run.

ember.cpp describes a model as a graph document (embed nodes, block nodes, head nodes, a state
declaration; graph_ir.cpp:1076-1100) and lets a block list say per layer which node applies
(graph_ir.cpp:2379).  The same idea here, one level up: a `ModelSpec` names, layer by layer, a
mixer, a feed-forward, two norms and their arrangement, each with its sizes and constants as
parameters; `schedule` is the order in which layers run, which may name a layer twice or let an
application read the cache that an earlier application wrote.  An architecture is a function from
its configuration to a `ModelSpec` (config/base.py); nothing below this file knows its name.
"""
from __future__ import annotations

import dataclasses
from typing import Any


@dataclasses.dataclass(frozen=True)
class PartSpec:
    """One part: `kind` is looked up in the registry of its role; `prefix` is put before the
    part's tensor names; `params` are the constructor's keyword arguments."""
    kind: str
    prefix: str = ""
    params: dict[str, Any] = dataclasses.field(default_factory=dict)


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    """One layer's parts.  `block` names the arrangement (how norms, mixer, feed-forward and
    the residual stream are wired).  An arrangement with one shared norm leaves `norm2` None; one
    with more norms than two (norms after the mixer and after the feed-forward as well) names the
    others in `more_norms`, and its block receives them as keyword arguments of those names."""
    block: str
    norm1: PartSpec | None
    mixer: PartSpec
    norm2: PartSpec | None
    ffn: PartSpec
    more_norms: tuple[tuple[str, PartSpec], ...] = ()


@dataclasses.dataclass(frozen=True)
class Application:
    """One entry of the run order.  `layer` indexes `ModelSpec.layers`.  With `cache_of` = the
    index of an earlier entry of the schedule, this application's mixer writes no cache of its own
    and reads that entry's."""
    layer: int
    cache_of: int | None = None


@dataclasses.dataclass(frozen=True)
class ModelSpec:
    width: int
    vocab_size: int
    token_table: str                 # tensor name of the [vocab, width] embedding table
    position: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[Application, ...]
    final_norm: PartSpec
    head: str | None                 # tensor name of the [vocab, width] head; None: tied to the token table
    embedding_scale: float = 1.0     # the embedded rows are multiplied by this (a model that scales by sqrt(width))
    head_bias: str | None = None     # tensor name of a [vocab] bias added to the logits
    logit_cap: float | None = None   # logits become cap * tanh(logits / cap)
    table_init_std: float = 0.02     # random-weights mode: std of the token table and the head
    stop_token_ids: tuple[int, ...] = ()
    # tensors that a checkpoint may hold and the model does not use (regular expressions)
    ignored_tensors: tuple[str, ...] = ()
    # prefixes that a checkpoint's tensor names may carry in front of the names the parts use (a
    # wrapper module's name); a detail of the architecture's checkpoints, so it stands here
    strip_prefixes: tuple[str, ...] = ()

    def check(self) -> None:
        if not self.layers:
            raise ValueError("ModelSpec: no layers")
        for i, app in enumerate(self.schedule):
            if not 0 <= app.layer < len(self.layers):
                raise ValueError(f"ModelSpec: schedule[{i}] names layer {app.layer}, there are {len(self.layers)}")
            if app.cache_of is not None:
                if not 0 <= app.cache_of < i:
                    raise ValueError(f"ModelSpec: schedule[{i}].cache_of = {app.cache_of} must name an earlier entry")
                if self.schedule[app.cache_of].cache_of is not None:
                    raise ValueError(f"ModelSpec: schedule[{i}].cache_of = {app.cache_of} names an entry that itself "
                                     "reads another's cache")
