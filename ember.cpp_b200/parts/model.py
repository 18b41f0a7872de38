"""A decoder built from a ModelSpec: token table, position encoding, the layers in their run
order, final norm, head.

The order is ember.cpp's for every decoder it runs: embed nodes, the block nodes once per
layer, then the head nodes on the wanted rows only (graph_ir.cpp:3010-3066; rows trimmed before
the head :3049-3061): `h = norm(x_rows)`, `logits = h Whead^T` without bias, Whead being the
token table when the head is tied (graph_ir.cpp:624-628, 757-762).  What other decoders put
around that order is data of the spec, not code of a model: a factor on the embedded rows, a bias
on the logits, a cap on them (cap * tanh(logits / cap)); GPT-2 uses none of the three.
"""
from __future__ import annotations

import torch

from .base import WeightSpec, build_block, build_part
from .spec import ModelSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        spec.check()
        self.spec = spec
        self.position = build_part("position", spec.position)
        self.blocks = []
        for layer in spec.layers:
            norm = lambda part: None if part is None else build_part("norm", part)  # noqa: E731
            self.blocks.append(build_block(layer.block, norm(layer.norm1), build_part("mixer", layer.mixer), norm(layer.norm2),
                                           build_part("ffn", layer.ffn), {name: norm(part) for name, part in layer.more_norms}))
        self.final_norm = build_part("norm", spec.final_norm)
        self.table = None
        self.head = None
        self.head_bias = None

    # ------------------------------------------------------------------ tensors
    def all_parts(self):
        parts = [self.position]
        for b in self.blocks:
            parts += b.parts()
        return parts + [self.final_norm]

    def weight_specs(self) -> list[WeightSpec]:
        s = self.spec
        specs = [WeightSpec(s.token_table, (s.vocab_size, s.width), std=s.table_init_std)]
        if s.head is not None:
            specs.append(WeightSpec(s.head, (s.vocab_size, s.width), std=s.table_init_std))
        if s.head_bias is not None:
            specs.append(WeightSpec(s.head_bias, (s.vocab_size,), std=s.table_init_std))
        for p in self.all_parts():
            specs += p.weight_specs()
        seen: dict[str, WeightSpec] = {}
        for w in specs:
            if w.name in seen and seen[w.name].shape != w.shape:
                raise ValueError(f"tensor {w.name!r} is wanted with shapes {seen[w.name].shape} and {w.shape}")
            seen.setdefault(w.name, w)
        return list(seen.values())

    def load(self, tensors: dict, runtime) -> None:
        """`tensors`: name -> tensor as stored (checked by the loader against weight_specs())."""
        get = tensors.__getitem__
        self.table = runtime.table(get(self.spec.token_table))
        self.head = self.table if self.spec.head is None else runtime.table(get(self.spec.head))
        self.head_bias = None if self.spec.head_bias is None else runtime.vector(get(self.spec.head_bias))
        for p in self.all_parts():
            p.load(get, runtime)

    # ------------------------------------------------------------------ what the cache must hold
    def max_positions(self) -> int | None:
        return self.position.max_positions()

    def application_needs(self):
        """(cache need, state need) of each entry of the schedule; an entry that reads another's
        cache has no cache need of its own."""
        out = []
        for app in self.spec.schedule:
            mixer = self.blocks[app.layer].mixer
            need = None if app.cache_of is not None else mixer.cache_need()
            out.append((need, mixer.state_need()))
        return out

    # ------------------------------------------------------------------ one step
    def forward(self, ctx):
        """Runs the tokens of `ctx.plan` through every entry of the schedule and returns float32
        logits [wanted rows, vocab] (None if no row is wanted)."""
        plan, ops = ctx.plan, ctx.ops
        ids = getattr(plan, "device_ids", None)   # sampled ids on the device that this step's tokens are taken from
        if ids is not None:
            x = ops.embed(plan.tokens, plan.positions, self.table, self.position.embedding_table(),
                          token_src=plan.token_src, ids=ids)
        else:
            x = ops.embed(plan.tokens, plan.positions, self.table, self.position.embedding_table())
        if self.spec.embedding_scale != 1.0:
            x = ops.scale_cap(x, scale=self.spec.embedding_scale)
        for i, app in enumerate(ctx.apps):
            # (a hint for the kernels: the first matrix that the block after this one streams)
            following = ctx.apps[i + 1].layer if i + 1 < len(ctx.apps) else None
            ctx.next_weights = self.blocks[following].mixer.stream_weights()[:1] if following is not None else ()
            x = self.blocks[app.layer].forward(ctx, x, app)
        if plan.n_want == 0:
            return None
        rows = x if plan.wants_every_row else ops.gather_rows(x, plan.want_rows, plan.n_want)
        h = self.final_norm.forward(ctx, rows, ctx.dtype)
        logits = ops.linear(h, self.head, self.head_bias, out_dtype=torch.float32)
        if self.spec.logit_cap is not None:
            logits = ops.scale_cap(logits, cap=self.spec.logit_cap)
        return logits
