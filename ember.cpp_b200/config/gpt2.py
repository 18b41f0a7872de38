"""GPT-2's configuration, read from its own config.json keys.

ember.cpp reads the same quantities from GGUF metadata when it builds its GPT-2 graph:
`embedding_length`, `block_count`, `attention.head_count`, `context_length`,
`attention.layer_norm_epsilon` (graph_ir.cpp:573-574, 725-729); the feed-forward width comes from
the tensor's shape (graph_ir.cpp:2505) and the head is tied when the file has no `output.weight`
(graph_ir.cpp:624-628).  Here they come under their Hugging Face names.  Defaults are the ones a
GPT-2 config.json implies when a key is absent (`n_inner` null means four times the width).
"""
from __future__ import annotations

import dataclasses
from typing import ClassVar

from .base import ConfigError, ModelConfig

# activation_function values and the form of GELU they mean.  ember.cpp's GPT-2 graph always
# uses the tanh form (graph_ir.cpp:745) and knows the erf form as `approx: none`
# (graph_ir.cpp:1257-1260); other activations are refused by name.
GELU_FORMS = {"gelu_new": "tanh", "gelu_pytorch_tanh": "tanh", "gelu_fast": "tanh", "gelu": "erf"}


@dataclasses.dataclass(frozen=True)
class GPT2Config(ModelConfig):
    architecture: ClassVar[str] = "GPT2LMHeadModel"
    aliases: ClassVar[dict[str, str]] = {"n_ctx": "n_positions"}

    vocab_size: int
    n_positions: int
    n_embd: int
    n_layer: int
    n_head: int
    n_inner: int | None = None
    activation_function: str = "gelu_new"
    layer_norm_epsilon: float = 1e-5
    tie_word_embeddings: bool = True
    scale_attn_weights: bool = True
    scale_attn_by_inverse_layer_idx: bool = False
    bos_token_id: int | None = None
    eos_token_id: int | None = None

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def inner(self) -> int:
        return self.n_inner if self.n_inner is not None else 4 * self.n_embd

    def validate(self) -> None:
        for key in ("vocab_size", "n_positions", "n_embd", "n_layer", "n_head"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"GPT2Config: {key} = {getattr(self, key)} must be positive")
        if self.n_inner is not None and self.n_inner <= 0:
            raise ConfigError(f"GPT2Config: n_inner = {self.n_inner} must be positive (or null for 4*n_embd)")
        if self.n_embd % self.n_head:
            raise ConfigError(f"GPT2Config: n_embd = {self.n_embd} is not a multiple of n_head = {self.n_head}")
        if self.activation_function not in GELU_FORMS:
            raise ConfigError(f"GPT2Config: activation_function = {self.activation_function!r} is not one of "
                              f"{sorted(GELU_FORMS)}")
        if not self.layer_norm_epsilon > 0:
            raise ConfigError(f"GPT2Config: layer_norm_epsilon = {self.layer_norm_epsilon} must be positive")
        for key in ("bos_token_id", "eos_token_id"):
            v = getattr(self, key)
            if v is not None and not 0 <= v < self.vocab_size:
                raise ConfigError(f"GPT2Config: {key} = {v} is outside the vocabulary [0, {self.vocab_size})")

    def check_dtype(self, dtype: str) -> None:
        """Refuses, before any weight is read, a model that the kernels of `dtype` cannot run; the
        error names the keys.  The true 32-bit path takes every size the configuration allows (head
        sizes up to 256); the bfloat16 kernels read rows in 16-byte pieces."""
        if self.head_dim > 256:
            raise ConfigError(f"GPT2Config: n_embd / n_head = {self.head_dim}: the attention kernels take head sizes up to 256")
        if dtype in ("bfloat16", "bf16"):
            if self.head_dim % 16:
                raise ConfigError(f"GPT2Config: n_embd / n_head = {self.n_embd} / {self.n_head} = {self.head_dim} is not a "
                                  "multiple of 16, which the bfloat16 attention kernels need; --dtype float32 runs this model")
            if self.inner % 8:
                raise ConfigError(f"GPT2Config: n_inner = {self.inner} is not a multiple of 8 (rows of 16 bytes), which the "
                                  "bfloat16 products need; --dtype float32 runs this model")
