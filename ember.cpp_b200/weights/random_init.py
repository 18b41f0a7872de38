"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration and
a seed.

ember.cpp has no such mode (its timing models come from an outside generator, and its parity
scripts initialise a tiny model of the family, tools/thirdparty_ember_check.py:57-74).  Each tensor
is drawn from N(mean, std) as its part declares (matrices and tables N(0, 0.02), the two output
projections with std 0.02/sqrt(2*layers), biases N(0, 0.01), norm gains 1 + N(0, 0.02), norm
biases N(0, 0.02)), from a generator keyed by the seed and the tensor's name, so a tensor's values
do not depend on which other tensors the model has.
"""
from __future__ import annotations

import json
import os
import zlib

import torch

from ..config.base import ModelConfig, get_architecture
from ..parts.base import WeightSpec
from ..parts.model import DecoderModel
from .safetensors_io import write_file


def _generator(seed: int, name: str, device="cpu") -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed((int(seed) * 0x9E3779B1 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF)
    return g


def random_tensor(spec: WeightSpec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    """Drawn on `device`; the values of a seed are those of that device's generator (a model
    folder is always written from the CPU's)."""
    if spec.integer:
        raise ValueError(f"random weights: no rule for the integer table {spec.name!r}")
    t = torch.empty(spec.shape, dtype=torch.float32, device=device)
    t.normal_(spec.mean, spec.std, generator=_generator(seed, spec.name, device))
    return t.to(dtype)


def random_tensors(specs: list[WeightSpec], seed: int, dtype: torch.dtype = torch.bfloat16,
                   device="cpu") -> dict[str, torch.Tensor]:
    return {s.name: random_tensor(s, seed, dtype, device) for s in specs}


def write_random_model(folder: str, config: ModelConfig, seed: int, dtype: torch.dtype = torch.bfloat16) -> str:
    """Writes `<folder>/config.json` and `<folder>/model.safetensors`; returns the folder."""
    arch = get_architecture(config.architecture)
    model = DecoderModel(arch.build_spec(config))
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=1)
    write_file(os.path.join(folder, "model.safetensors"), random_tensors(model.weight_specs(), seed, dtype),
               {"format": "pt", "seed": str(seed)})
    return folder
