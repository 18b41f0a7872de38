"""A small model library with generation of its own for one GPU: everything between a request's
tokens and its next token, built from parts so that another architecture is a new ModelSpec.

The folder's name has a dot in it, so it is imported under the name `ember_cpp_b200` through the
module of that name beside this folder.
"""
from . import config, parts, weights, cache  # noqa: F401
from . import architectures  # noqa: F401  (registers the built-in architectures)
from .config import ConfigError, GPT2Config, load_config, register_architecture
from .parts import ModelSpec, register_part
from .engine import Engine, StepError
from .engine.generate import Generation, GenerationParams, Generator
from .sampling import Sampler, SamplingParams
from .api import Session, TinyLlamaSession
from .weights import WeightError, write_random_model
from .options import OptionError, RuntimeOptions

__all__ = ["ConfigError", "Engine", "GPT2Config", "Generation", "GenerationParams", "Generator", "ModelSpec", "OptionError",
           "RuntimeOptions", "Sampler",
           "SamplingParams", "Session", "StepError", "TinyLlamaSession", "WeightError", "load_config",
           "register_architecture", "register_part", "write_random_model"]
