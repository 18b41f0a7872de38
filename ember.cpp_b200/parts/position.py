"""Position encodings.

GPT-2 adds a learned row per absolute position to the token embedding:
`x[t,:] += wpe[P+t,:]`, and a position past the table is an error (graph_ir.cpp:2410-2420;
kernel graph_ir_cuda.cu:26-32).  The table bounds the context.  `none` is the encoding of a model
whose mixers carry position themselves.
"""
from __future__ import annotations

from .base import Position, WeightSpec, register_part


class LearnedAbsolute(Position):

    def __init__(self, prefix: str, width: int, n_positions: int, table: str = "weight", init_std: float = 0.02):
        super().__init__(prefix)
        self.width, self.n_positions = int(width), int(n_positions)
        self.table_name = prefix + table
        self.init_std = init_std
        self.table = None

    def weight_specs(self):
        return [WeightSpec(self.table_name, (self.n_positions, self.width), std=self.init_std)]

    def load(self, get, runtime):
        self.table = runtime.table(get(self.table_name))

    def embedding_table(self):
        return self.table

    def max_positions(self):
        return self.n_positions


class NoPosition(Position):

    def __init__(self, prefix: str = ""):
        super().__init__(prefix)


register_part("position", "learned_absolute", LearnedAbsolute)
register_part("position", "none", NoPosition)
