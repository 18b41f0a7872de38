"""Weights by tensor name, checked against what the model's parts ask for.

ember.cpp binds every tensor that its graph names and stops at the first that is missing
("IR weight 'X' is not in the GGUF", graph_ir.cpp:1899; "Tensor not found in SafeTensorsLoader
metadata", safetensors_loader.cpp:506-512) or whose width does not fit (graph_ir.cpp:2502-2504).
Here the whole table is checked at once: one error lists every missing tensor, every unexpected
one and every wrong shape.
"""
from __future__ import annotations

import re

import torch

from ..parts.base import WeightSpec
from .safetensors_io import UnreadTensor, read_folder


class WeightError(ValueError):
    """Missing, unexpected or misshapen tensors; `missing`, `unexpected`, `wrong_shape` list them."""

    def __init__(self, where: str, missing, unexpected, wrong_shape, wrong_type=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_type = list(wrong_shape), list(wrong_type)
        lines = [f"{where}: the tensors do not fit the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        for name, got in self.wrong_type:
            lines.append(f"  wrong type: {name} is {got}")
        super().__init__("\n".join(lines))


def _strip(name: str, prefixes) -> str:
    for p in prefixes:
        if name.startswith(p):
            return name[len(p):]
    return name


def check_tensors(where: str, tensors: dict[str, torch.Tensor], specs: list[WeightSpec], ignored=(),
                  strip_prefixes=()) -> dict[str, torch.Tensor]:
    """Returns name -> tensor for exactly the wanted names, or raises one WeightError.  `ignored`
    and `strip_prefixes` come from the architecture's ModelSpec.  A tensor whose stored type the
    reader does not know (`UnreadTensor`) is an error only if the model wants it."""
    have = {_strip(k, strip_prefixes): v for k, v in tensors.items()}
    want = {s.name: s for s in specs}
    missing = [n for n in want if n not in have]
    patterns = [re.compile(p) for p in ignored]
    unexpected = [n for n in have if n not in want and not any(p.fullmatch(n) for p in patterns)]
    wrong_shape = [(n, want[n].shape, tuple(have[n].shape)) for n in want
                   if n in have and tuple(have[n].shape) != tuple(want[n].shape)]
    wrong_type = []
    for n, s in want.items():
        if n in have and isinstance(have[n], UnreadTensor):
            wrong_type.append((n, f"stored as {have[n].dtype_name}, which this library does not read"))
        elif n in have:
            is_int = not have[n].dtype.is_floating_point
            if is_int != s.integer:
                wrong_type.append((n, f"{have[n].dtype}, expected {'an integer' if s.integer else 'a floating'} type"))
    if missing or unexpected or wrong_shape or wrong_type:
        raise WeightError(where, sorted(missing), sorted(unexpected), sorted(wrong_shape), sorted(wrong_type))
    return {n: have[n] for n in want}


def load_checked(folder: str, specs: list[WeightSpec], ignored=(), strip_prefixes=()) -> dict[str, torch.Tensor]:
    return check_tensors(folder, read_folder(folder), specs, ignored, strip_prefixes)
