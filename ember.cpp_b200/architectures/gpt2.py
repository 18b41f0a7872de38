"""GPT-2 (`GPT2LMHeadModel`) as a ModelSpec.

The graph that ember.cpp builds for `general.architecture = gpt2` (graph_ir.cpp:721-766):
token embedding plus learned positions; per layer LayerNorm, fused biased qkv, causal attention
with scale 1/sqrt(head size), biased output projection, residual, LayerNorm, biased up projection,
GELU (tanh form), biased down projection, residual; then LayerNorm and a head tied to the token
table unless the file carries one.  Tensor names are the Hugging Face ones; the four block
matrices are stored [in, out] (Conv1D) and are transposed once at load.
`scale_attn_by_inverse_layer_idx` is not in ember.cpp: it divides the scale by layer + 1.
"""
from __future__ import annotations

import math

from ..config.base import register_architecture
from ..config.gpt2 import GELU_FORMS, GPT2Config
from ..parts.spec import Application, LayerSpec, ModelSpec, PartSpec


def build_spec(cfg: GPT2Config) -> ModelSpec:
    d, hd = cfg.n_embd, cfg.head_dim
    # random-weights mode: both output projections are drawn with std / sqrt(2 * n_layer)
    proj_std = 0.02 / math.sqrt(2 * cfg.n_layer)
    layers = []
    for i in range(cfg.n_layer):
        scale = 1.0 / math.sqrt(hd) if cfg.scale_attn_weights else 1.0
        if cfg.scale_attn_by_inverse_layer_idx:
            scale /= i + 1
        p = f"h.{i}."
        layers.append(LayerSpec(
            block="pre_norm",
            norm1=PartSpec("layernorm", p + "ln_1.", {"width": d, "eps": cfg.layer_norm_epsilon}),
            mixer=PartSpec("causal_attention", p + "attn.", {
                "width": d, "n_heads": cfg.n_head, "kv_heads": cfg.n_head, "head_dim": hd, "scale": scale,
                "qkv": "c_attn", "out": "c_proj", "stored": "in_out", "bias": True, "out_init_std": proj_std}),
            norm2=PartSpec("layernorm", p + "ln_2.", {"width": d, "eps": cfg.layer_norm_epsilon}),
            ffn=PartSpec("dense", p + "mlp.", {
                "width": d, "inner": cfg.inner, "activation": "gelu_" + GELU_FORMS[cfg.activation_function],
                "up": "c_fc", "down": "c_proj", "stored": "in_out", "bias": True, "down_init_std": proj_std}),
        ))
    return ModelSpec(
        width=d,
        vocab_size=cfg.vocab_size,
        token_table="wte.weight",
        position=PartSpec("learned_absolute", "wpe.", {"width": d, "n_positions": cfg.n_positions}),
        layers=tuple(layers),
        schedule=tuple(Application(i) for i in range(cfg.n_layer)),
        final_norm=PartSpec("layernorm", "ln_f.", {"width": d, "eps": cfg.layer_norm_epsilon}),
        head=None if cfg.tie_word_embeddings else "lm_head.weight",
        stop_token_ids=() if cfg.eos_token_id is None else (cfg.eos_token_id,),
        # buffers that GPT-2 checkpoints carry and that are no parameters; a tied checkpoint may
        # also repeat the token table as lm_head.weight
        ignored_tensors=(r"h\.\d+\.attn\.bias", r"h\.\d+\.attn\.masked_bias") +
                        ((r"lm_head\.weight",) if cfg.tie_word_embeddings else ()),
        # GPT2LMHeadModel keeps its blocks in a module named `transformer`
        strip_prefixes=("transformer.",),
    )


register_architecture(GPT2Config.architecture, GPT2Config, build_spec)
