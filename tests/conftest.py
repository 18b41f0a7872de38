"""Shared fixtures: the two tiny GPT-2 configurations, model folders made in temporary folders,
and the `gpu` marker.

The two configurations differ in every size and option: layers 2/3, width 64/96, heads 4/3, head
size 16/32, inner 256 (4x) / 320 (not 4x), vocabulary 512/1000, positions 128/96, eps 1e-5/1e-6,
tanh/erf GELU, tied/untied head, inverse-layer attention scale off/on.
"""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

TINY = {
    "tiny_a": dict(vocab_size=512, n_positions=128, n_embd=64, n_layer=2, n_head=4, n_inner=256,
                   activation_function="gelu_new", layer_norm_epsilon=1e-5, tie_word_embeddings=True),
    "tiny_b": dict(vocab_size=1000, n_positions=96, n_embd=96, n_layer=3, n_head=3, n_inner=320,
                   activation_function="gelu", layer_norm_epsilon=1e-6, tie_word_embeddings=False,
                   scale_attn_by_inverse_layer_idx=True),
}
SEEDS = {"tiny_a": 0, "tiny_b": 1}

# relative to the range of the reference row: max|delta| / (max - min), as ember.cpp's own gates
# measure it (tools/thirdparty_ember_check.py:78-80).  float32: its CUDA-vs-CPU gate allows 1e-4
# and its CPU-vs-HF gate 1e-5 (tools/ir_device_gate.cpp:158-191); here the tighter one.
# bfloat16: the plain implementation with its activations rounded to bfloat16 at the same places
# moves by about 1e-3 of the range on these models; an engine in bfloat16 may differ from the exact
# result by a small multiple of that.
TOL = {"float32": 1e-5, "bfloat16": 8e-3}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (sm_100a) and the built kernels")


def rel_error(got: np.ndarray, ref: np.ndarray) -> float:
    """Worst row of max|delta| / (max - min of the reference row)."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    if ref.ndim == 1:
        got, ref = got[None], ref[None]
    span = ref.max(axis=-1) - ref.min(axis=-1)
    return float((np.abs(got - ref).max(axis=-1) / span).max())


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    """name -> model folder (config.json, model.safetensors) with random weights in bfloat16."""
    import ember_cpp_b200 as E
    out = {}
    for name, cfg in TINY.items():
        folder = tmp_path_factory.mktemp(name)
        E.write_random_model(str(folder), E.GPT2Config.from_dict(cfg), SEEDS[name])
        out[name] = str(folder)
    return out


@pytest.fixture(scope="session")
def plains(tiny_folders):
    import plain_gpt2
    return {name: plain_gpt2.PlainGPT2(folder) for name, folder in tiny_folders.items()}


def random_ids(seed: int, vocab: int, n: int) -> list:
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def run_batch(engine, sequences, prompt_lengths):
    """Feeds given sequences as one batch: the first `prompt_lengths[i]` tokens of each in one step,
    then one token each per step; a sequence leaves (its slot closed) when its tokens are used up.
    Returns (per sequence: float32 logits [len, vocab] of every position, the slots used)."""
    slots = [engine.open() for _ in sequences]
    rows = [[] for _ in sequences]
    out = engine.step([(s, seq[:n], list(range(n))) for s, seq, n in zip(slots, sequences, prompt_lengths)])
    out = out.detach().cpu().numpy()
    at = 0
    for i, n in enumerate(prompt_lengths):
        rows[i].extend(out[at:at + n])
        at += n
    fed = list(prompt_lengths)
    live = [i for i in range(len(sequences)) if fed[i] < len(sequences[i])]
    for i in range(len(sequences)):
        if i not in live:
            engine.close(slots[i])
    while live:
        out = engine.step([(slots[i], [sequences[i][fed[i]]], [0]) for i in live]).detach().cpu().numpy()
        for r, i in enumerate(live):
            rows[i].append(out[r])
            fed[i] += 1
        for i in [i for i in live if fed[i] == len(sequences[i])]:
            engine.close(slots[i])
        live = [i for i in live if fed[i] < len(sequences[i])]
    return [np.stack(r) for r in rows], slots
