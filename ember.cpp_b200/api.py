"""The Python entry point, in the manner of ember.cpp's `TinyLlamaSession`.

ember.cpp's binding: `TinyLlamaSession(model_path, tokenizer_path, threads=1, n_gpu_layers=0,
use_mmap=True, use_kv_quant=False, use_batch_generation=False, max_batch_size=1)` with
`.generate(prompt, steps=128, temperature=0.1, top_k=40, top_p=0.9, system_prompt="",
apply_q_a_format=True)`, `.generate_batch(prompts, ...)` and `.get_config()`
(bindings.cpp:109-304).  The names and meanings are kept where they apply.  What differs: this
library works on token ids (it has no tokenizer), so a prompt is a list of ids and the reply is a
list of ids; it runs on one GPU only, so `n_gpu_layers` may be -1 (all) and nothing else;
quantised caches are not built, so `use_kv_quant` must stay False.  `dtype` and `max_tokens` (the
cache's size in positions) are additions, and so is `options` (a RuntimeOptions: every switch of
the runtime in one struct; dtype and max_tokens given here override its fields).
"""
from __future__ import annotations

from typing import Callable, Sequence

from .engine.engine import Engine
from .engine.generate import Generation, GenerationParams, Generator
from .sampling.sampler import SamplingParams


class Session:
    def __init__(self, model_path: str, tokenizer_path: str | None = None, threads: int = 1, n_gpu_layers: int = -1,
                 use_mmap: bool = True, use_kv_quant: bool = False, use_batch_generation: bool = True,
                 max_batch_size: int = 8, dtype: str | None = None, max_tokens: int | None = None, seed: int = 0,
                 ops=None, device: str = "cuda", options=None):
        if n_gpu_layers != -1:
            raise ValueError("n_gpu_layers: this library runs every layer on the GPU (-1); it has no CPU path")
        if use_kv_quant:
            raise ValueError("use_kv_quant: quantised caches are not built")
        if max_batch_size <= 0:
            raise ValueError(f"max_batch_size = {max_batch_size} must be positive")
        self.model_path, self.max_batch_size, self.seed = str(model_path), int(max_batch_size), int(seed)
        self.use_batch_generation = bool(use_batch_generation)
        if max_tokens is None:
            from .config.base import load_config
            from .config.base import get_architecture
            from .parts.model import DecoderModel
            cfg = load_config(self.model_path)
            positions = DecoderModel(get_architecture(cfg.architecture).build_spec(cfg)).max_positions() or 4096
            max_tokens = self.max_batch_size * (-(-positions // 64) * 64)
        self._attach(Engine.from_folder(self.model_path, dtype=dtype, max_tokens=max_tokens, ops=ops, device=device,
                                        options=options))

    def _attach(self, engine: Engine) -> None:
        self.engine = engine
        self.generator = Generator(engine)
        self._callback: Callable[[int, int], None] | None = None
        self._served = 0

    @classmethod
    def from_engine(cls, engine: Engine, max_batch_size: int = 8, seed: int = 0) -> "Session":
        """A session over an engine that already exists (a model built from a spec, or shared)."""
        self = cls.__new__(cls)
        self.model_path, self.max_batch_size, self.seed = "", int(max_batch_size), int(seed)
        self.use_batch_generation = True
        self._attach(engine)
        return self

    # ------------------------------------------------------------------ ember.cpp's surface
    def get_config(self):
        return self.engine.config

    def set_seed(self, seed: int) -> None:
        """ember.cpp: api.h:240."""
        self.seed = int(seed)
        self._served = 0

    def set_token_callback(self, callback: Callable[[int, int], None] | None) -> None:
        """`callback(request index, token)` for every new token (ember.cpp: api.h:243)."""
        self._callback = callback

    def generate(self, prompt: Sequence[int], steps: int = 128, temperature: float = 0.1, top_k: int = 40,
                 top_p: float = 0.9, stop_token_ids: Sequence[int] | None = None) -> list[int]:
        """New token ids for one prompt of token ids; `steps` is the most new tokens."""
        return self.generate_batch([prompt], steps, temperature, top_k, top_p, stop_token_ids)[0]

    def generate_batch(self, prompts: Sequence[Sequence[int]], steps: int = 128, temperature: float = 0.1,
                       top_k: int = 40, top_p: float = 0.9, stop_token_ids: Sequence[int] | None = None) -> list[list[int]]:
        return [g.tokens for g in self.generate_detailed(prompts, steps, temperature, top_k, top_p, stop_token_ids)]

    # ------------------------------------------------------------------ with finish reasons
    def generate_detailed(self, prompts, steps=128, temperature=0.1, top_k=40, top_p=0.9,
                          stop_token_ids=None) -> list[Generation]:
        params = GenerationParams(
            max_new_tokens=int(steps),
            sampling=SamplingParams(float(temperature), int(top_k), float(top_p), self.seed),
            stop_token_ids=None if stop_token_ids is None else tuple(int(t) for t in stop_token_ids),
            max_batch_size=self.max_batch_size if self.use_batch_generation else 1)
        out = self.generator.generate([list(p) for p in prompts], params, self._callback, first_stream=self._served)
        self._served += len(prompts)
        return out


# ember.cpp's class name, for callers that switch over
TinyLlamaSession = Session
