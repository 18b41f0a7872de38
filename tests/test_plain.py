"""The plain implementation itself (no GPU): against logits of ember.cpp's own CPU interpreter
(tests/golden/*.npz, made by tests/golden/make_golden.py), and each part against an independent
restatement in torch."""
import hashlib
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_gpt2
from conftest import rel_error

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_plain_equals_embers_interpreter(tiny_folders, plains, name):
    """ember.cpp's interpreter ran the same weights (configuration A on the graph it builds itself,
    B on that graph edited for the erf GELU, the untied head and the per-layer scale).  Its own
    gates accept 1e-5 of the logit range against outside references and the same top-1
    (tools/thirdparty_ember_check.py:204-210)."""
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    with open(os.path.join(tiny_folders[name], "model.safetensors"), "rb") as f:
        digest = hashlib.sha256(f.read()).hexdigest()
    assert digest == bytes(g["weights_sha256"]).decode(), \
        "the random-weights mode no longer writes the bytes the golden files were made from; run make_golden.py again"
    assert json.loads(bytes(g["config"]).decode())["n_embd"] == plains[name].n_embd
    for i in range(3):
        ids = g[f"ids{i}"].tolist()
        ref = g[f"prefill{i}"]
        got = plains[name].logits(ids)
        assert rel_error(got, ref) < 1e-5
        assert (got.argmax(-1) == ref.argmax(-1)).all()
        assert bool(g[f"decode_equals_prefill{i}"])


def test_layer_norm():
    rng = np.random.default_rng(0)
    x, w, b = rng.normal(size=(5, 48)) * 3 + 1, rng.normal(size=48), rng.normal(size=48)
    want = torch.nn.functional.layer_norm(torch.tensor(x), (48,), torch.tensor(w), torch.tensor(b), 1e-6).numpy()
    assert np.allclose(plain_gpt2.layer_norm(x, w, b, 1e-6), want, atol=1e-12)


def test_gelu_forms():
    x = np.linspace(-6, 6, 101)
    assert np.allclose(plain_gpt2.gelu(x, "tanh"), torch.nn.functional.gelu(torch.tensor(x), approximate="tanh").numpy(),
                       atol=1e-12)
    assert np.allclose(plain_gpt2.gelu(x, "erf"), torch.nn.functional.gelu(torch.tensor(x)).numpy(), atol=1e-12)
    assert plain_gpt2.gelu_form("gelu_new") == "tanh" and plain_gpt2.gelu_form("gelu") == "erf"
    with pytest.raises(ValueError):
        plain_gpt2.gelu_form("relu")


@pytest.mark.parametrize("heads, kv_heads, window", [(4, 4, 0), (6, 2, 0), (3, 3, 5), (4, 1, 9)])
def test_attention(heads, kv_heads, window):
    rng = np.random.default_rng(1)
    T, hd = 23, 8
    q = rng.normal(size=(T, heads * hd))
    k, v = rng.normal(size=(T, kv_heads * hd)), rng.normal(size=(T, kv_heads * hd))
    got = plain_gpt2.attention(q, k, v, heads, kv_heads, hd, 0.3, window)
    tq = torch.tensor(q).view(T, heads, hd).transpose(0, 1)
    tk = torch.tensor(k).view(T, kv_heads, hd).transpose(0, 1).repeat_interleave(heads // kv_heads, 0)
    tv = torch.tensor(v).view(T, kv_heads, hd).transpose(0, 1).repeat_interleave(heads // kv_heads, 0)
    s = tq @ tk.transpose(1, 2) * 0.3
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    mask = (j <= i) & ((j > i - window) if window else True)
    s = s.masked_fill(~mask, float("-inf"))
    want = (torch.softmax(s, -1) @ tv).transpose(0, 1).reshape(T, heads * hd).numpy()
    assert np.allclose(got, want, atol=1e-12)


def test_embedding_and_positions():
    wte, wpe = np.arange(20.0).reshape(5, 4), np.arange(12.0).reshape(3, 4) * 100
    x = plain_gpt2.position_embedding(plain_gpt2.token_embedding(wte, [4, 0]), wpe, 1)
    assert x.tolist() == [[416, 517, 618, 719], [800, 901, 1002, 1103]]
    with pytest.raises(ValueError):
        plain_gpt2.token_embedding(wte, [5])
    with pytest.raises(ValueError):
        plain_gpt2.position_embedding(np.zeros((3, 4)), wpe, 1)


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.0e-40, 65504.0, 1.0 + 2 ** -8])
    want = torch.tensor(x, dtype=torch.float32).to(torch.bfloat16).to(torch.float64).numpy()
    assert np.array_equal(plain_gpt2.round_bf16(x), want)


def test_sampler_rules():
    row = np.log(np.array([0.05, 0.4, 0.05, 0.3, 0.2]))
    assert plain_gpt2.sample(row, 0.0, 40, 0.9, 0.99) == 1                    # below 0.05: first maximum
    assert plain_gpt2.sample(np.array([1.0, 3.0, 3.0]), 0.01, 0, 1.0, 0.5) == 1
    # top_k 2 keeps {1, 3}; drawn in index order with weights 0.4 : 0.3
    assert [plain_gpt2.sample(row, 1.0, 2, 1.0, u) for u in (0.0, 0.5, 0.58, 0.99)] == [1, 1, 3, 3]
    # top_p 0.6: 0.4 + 0.3 reaches it -> {1, 3}; top_p 0.75 needs the third -> {1, 3, 4}
    assert {plain_gpt2.sample(row, 1.0, 0, 0.6, u) for u in np.linspace(0, 0.999, 50)} == {1, 3}
    assert {plain_gpt2.sample(row, 1.0, 0, 0.75, u) for u in np.linspace(0, 0.999, 50)} == {1, 3, 4}
    # ties at the edge of top_k go to the larger index first (pairs ordered by (p, index) descending)
    assert {plain_gpt2.sample(np.zeros(4), 1.0, 2, 1.0, u) for u in np.linspace(0, 0.999, 20)} == {2, 3}
    counts = np.bincount([plain_gpt2.sample(row, 1.0, 0, 1.0, plain_gpt2.uniform01(3, 0, c)) for c in range(4000)],
                         minlength=5) / 4000
    assert np.abs(counts - np.exp(row)).max() < 0.03
    us = [plain_gpt2.uniform01(1, s, c) for s in range(20) for c in range(50)]
    assert 0 <= min(us) and max(us) < 1 and abs(np.mean(us) - 0.5) < 0.03 and len(set(us)) > 990


def test_uniform_matches_the_librarys():
    from ember_cpp_b200.sampling import uniform01
    for args in [(0, 0, 0), (7, 3, 11), (2 ** 40, 5, 2 ** 20)]:
        assert uniform01(*args) == plain_gpt2.uniform01(*args)


def test_generate_stops(plains):
    plain = plains["tiny_a"]
    prompt = [1, 2, 3]
    free, why = plain_gpt2.generate(plain, prompt, 5, 1.0, 0, 1.0, seed=4)
    assert why == "length" and len(free) == 5
    cut, why = plain_gpt2.generate(plain, prompt, 5, 1.0, 0, 1.0, seed=4, stop_ids=(free[2],))
    assert why == "stop" and cut == free[:free.index(free[2]) + 1]
    full = list(range(plain.n_positions))
    out, why = plain_gpt2.generate(plain, full, 5)
    assert why == "context" and len(out) == 1
