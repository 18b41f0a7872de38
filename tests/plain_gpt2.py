"""Plain GPT-2: whole sequences, no cache, one function for each part.

Written from the formulas of ember.cpp's graph interpreter (its CPU form), which is how that
project runs GPT-2.  Nothing here is shared with the engine: it has its own safetensors reader,
its own arithmetic (numpy, float64 unless asked otherwise) and no notion of steps, slots or pages.
Every function cites the file and lines of ember.cpp that give its formula.

Where ember.cpp accumulates in float64 and rounds to float32 (layer norm statistics, dot
products), this file simply stays in float64: it is the exact value that both the reference
and the engine approximate.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np

# --------------------------------------------------------------------------- model folder


def _bf16_to_f32(raw: np.ndarray) -> np.ndarray:
    return (raw.astype(np.uint32) << 16).view(np.float32)


def read_safetensors(path: str) -> dict[str, np.ndarray]:
    """8-byte little-endian header length, JSON header, data block
    (safetensors_loader.cpp:151-164; per tensor dtype/shape/data_offsets :459-475)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        buf = data[b:e]
        dt = meta["dtype"].upper()
        if dt == "F32":
            a = np.frombuffer(buf, dtype="<f4").astype(np.float64)
        elif dt == "BF16":
            a = _bf16_to_f32(np.frombuffer(buf, dtype="<u2")).astype(np.float64)
        elif dt == "F16":
            a = np.frombuffer(buf, dtype="<f2").astype(np.float64)
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name}")
        out[name] = a.reshape(meta["shape"])
    return out


class PlainGPT2:
    """Config values and weights of one model folder, as float64 arrays under HF names."""

    def __init__(self, folder: str):
        with open(os.path.join(folder, "config.json")) as f:
            c = json.load(f)
        self.cfg = c
        self.n_layer = c["n_layer"]
        self.n_embd = c["n_embd"]
        self.n_head = c["n_head"]
        self.n_inner = c.get("n_inner") or 4 * self.n_embd
        self.vocab = c["vocab_size"]
        self.n_positions = c.get("n_positions", c.get("n_ctx"))
        self.eps = c.get("layer_norm_epsilon", 1e-5)
        self.act = c.get("activation_function", "gelu_new")
        self.tied = c.get("tie_word_embeddings", True)
        self.inv_layer_scale = c.get("scale_attn_by_inverse_layer_idx", False)
        self.scale_attn = c.get("scale_attn_weights", True)
        w = read_safetensors(os.path.join(folder, "model.safetensors"))
        self.w = {(k[len("transformer."):] if k.startswith("transformer.") else k): v for k, v in w.items()}

    # ----------------------------------------------------------------------- whole model
    def logits(self, ids, round_to=None) -> np.ndarray:
        """Logits [T, vocab] of one whole sequence.  `round_to="bfloat16"` rounds the activations
        at the places where the serving path stores them in bfloat16."""
        return forward(self, list(ids), round_to)


# --------------------------------------------------------------------------- parts


def round_bf16(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to bfloat16 (a test aid: the places where a serving path may store
    16-bit activations)."""
    f = a.astype(np.float32).view(np.uint32).astype(np.uint64)
    r = ((f + 0x7FFF + ((f >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).astype(np.float64)


def _maybe_round(a, round_to):
    return round_bf16(a) if round_to == "bfloat16" else a


def token_embedding(wte: np.ndarray, ids) -> np.ndarray:
    """x[t,:] = wte[id_t,:]; an id outside [0, vocab) is an error (graph_ir.cpp:2381-2409)."""
    for i in ids:
        if i < 0 or i >= wte.shape[0]:
            raise ValueError(f"token id {i} out of range")
    return wte[np.asarray(ids, dtype=np.int64)].copy()


def position_embedding(x: np.ndarray, wpe: np.ndarray, start: int = 0) -> np.ndarray:
    """x[t,:] += wpe[start+t,:] (graph_ir.cpp:2410-2420)."""
    T = x.shape[0]
    if start + T > wpe.shape[0]:
        raise ValueError(f"position {start + T - 1} exceeds the table")
    return x + wpe[start:start + T]


def layer_norm(x: np.ndarray, w: np.ndarray, b: np.ndarray, eps: float) -> np.ndarray:
    """mean, biased variance in two passes, (x-mean)/sqrt(var+eps)*w+b (graph_ir.cpp:2421-2439)."""
    mean = x.sum(axis=-1, keepdims=True) / x.shape[-1]
    var = ((x - mean) ** 2).sum(axis=-1, keepdims=True) / x.shape[-1]
    return (x - mean) * (1.0 / np.sqrt(var + eps)) * w + b


def linear(x: np.ndarray, w_out_in: np.ndarray, bias: np.ndarray | None) -> np.ndarray:
    """Y[t,o] = dot(W[o,:], X[t,:]) then + bias as a second pass
    (graph_ir.cpp:2498-2520; utils.cpp:867-909; cpu_dot.h:13-21)."""
    y = x @ w_out_in.T
    return y if bias is None else y + bias


def conv1d_weight(w_in_out: np.ndarray) -> np.ndarray:
    """GPT-2 checkpoints store the four block matrices as [in, out]; the reference binds
    [out, in] rows (graph_ir.h:8), so the stored matrix is transposed."""
    return w_in_out.T


def split_qkv(qkv: np.ndarray, n_head: int, kv_heads: int, head_dim: int):
    """Columns [0,H*hd) | [H*hd, +KV*hd) | [.., +KV*hd) in that order
    (graph_ir.cpp:734 sizes; :2440-2470)."""
    a = n_head * head_dim
    b = a + kv_heads * head_dim
    return qkv[:, :a], qkv[:, a:b], qkv[:, b:]


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, n_head: int, kv_heads: int, head_dim: int,
              scale: float, window: int = 0) -> np.ndarray:
    """Causal attention of T query rows over the same T key rows, positions 0..T-1.

    s_j = (q.k_j)*scale for j <= t; softmax with the row maximum subtracted; a = sum_j p_j v_j
    (cpu_attention.cpp:92-211; softmax utils.cpp:670-693, whose 1e-9 in the denominator is below
    half an ulp of a sum >= 1 and is left out).  Query head h reads key/value head
    h // (n_head // kv_heads) (cpu_attention.cpp:127).  With window > 0 a query at p sees
    positions p-window+1 .. p (cpu_attention.cpp swa_visible_ranges, win_lo)."""
    T = q.shape[0]
    out = np.zeros((T, n_head * head_dim))
    group = n_head // kv_heads
    for h in range(n_head):
        g = h // group
        qh = q[:, h * head_dim:(h + 1) * head_dim]
        kh = k[:, g * head_dim:(g + 1) * head_dim]
        vh = v[:, g * head_dim:(g + 1) * head_dim]
        for t in range(T):
            lo = max(0, t + 1 - window) if window > 0 else 0
            s = (kh[lo:t + 1] @ qh[t]) * scale
            e = np.exp(s - s.max())
            p = e / e.sum()
            out[t, h * head_dim:(h + 1) * head_dim] = p @ vh[lo:t + 1]
    return out


def gelu(x: np.ndarray, form: str) -> np.ndarray:
    """tanh form 0.5 v (1 + tanh(sqrt(2/pi) (v + 0.044715 v^3))); erf form 0.5 v (1 + erf(v/sqrt 2))
    (graph_ir.cpp:2471-2481)."""
    if form == "tanh":
        c = math.sqrt(2.0 / math.pi)
        return 0.5 * x * (1.0 + np.tanh(c * (x + 0.044715 * x * x * x)))
    if form == "erf":
        erf = np.vectorize(math.erf)
        return 0.5 * x * (1.0 + erf(x / math.sqrt(2.0)))
    raise ValueError(form)


def gelu_form(activation_function: str) -> str:
    """GPT-2 graphs of the reference always use the tanh form (graph_ir.cpp:745); the erf form is
    its `approx: none` (graph_ir.cpp:1257-1260).  HF names map onto the two."""
    if activation_function in ("gelu_new", "gelu_pytorch_tanh", "gelu_fast"):
        return "tanh"
    if activation_function == "gelu":
        return "erf"
    raise ValueError(f"activation_function {activation_function!r}")


def mlp(h: np.ndarray, w_fc, b_fc, w_proj, b_proj, form: str, round_to=None) -> np.ndarray:
    """u = h Wup^T + b; u = gelu(u); f = u Wdown^T + b (graph_ir.cpp:743-746)."""
    u = linear(h, w_fc, b_fc)
    u = _maybe_round(gelu(u, form), round_to)
    return linear(u, w_proj, b_proj)


def block(m: PlainGPT2, layer: int, x: np.ndarray, round_to=None) -> np.ndarray:
    """x -> ln_1 -> c_attn -> split -> attention -> c_proj -> +x -> ln_2 -> c_fc -> gelu -> c_proj -> +x
    (graph_ir.cpp:732-756, the sequential-residual branch)."""
    w = m.w
    p = f"h.{layer}."
    hd = m.n_embd // m.n_head
    h = _maybe_round(layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], m.eps), round_to)
    qkv = _maybe_round(linear(h, conv1d_weight(w[p + "attn.c_attn.weight"]), w[p + "attn.c_attn.bias"]), round_to)
    q, k, v = split_qkv(qkv, m.n_head, m.n_head, hd)
    scale = (1.0 / math.sqrt(hd)) if m.scale_attn else 1.0  # graph_ir.cpp:741
    if m.inv_layer_scale:
        scale = scale / (layer + 1)  # not in the reference; GPT-2's scale_attn_by_inverse_layer_idx
    a = _maybe_round(attention(q, k, v, m.n_head, m.n_head, hd, scale), round_to)
    x = x + linear(a, conv1d_weight(w[p + "attn.c_proj.weight"]), w[p + "attn.c_proj.bias"])
    h2 = _maybe_round(layer_norm(x, w[p + "ln_2.weight"], w[p + "ln_2.bias"], m.eps), round_to)
    f = mlp(h2, conv1d_weight(w[p + "mlp.c_fc.weight"]), w[p + "mlp.c_fc.bias"],
            conv1d_weight(w[p + "mlp.c_proj.weight"]), w[p + "mlp.c_proj.bias"], gelu_form(m.act), round_to)
    return x + f


def lm_head(m: PlainGPT2, x: np.ndarray, round_to=None) -> np.ndarray:
    """h = LN(x; ln_f); logits = h Whead^T, no bias; Whead is lm_head.weight, or wte when tied
    (graph_ir.cpp:624-628, 757-762)."""
    h = _maybe_round(layer_norm(x, m.w["ln_f.weight"], m.w["ln_f.bias"], m.eps), round_to)
    wh = m.w["wte.weight"] if m.tied else m.w["lm_head.weight"]
    return linear(h, wh, None)


def forward(m: PlainGPT2, ids, round_to=None) -> np.ndarray:
    """embed -> L blocks -> ln_f -> head (experiments/gpt2_2026-10-25/ember_built.ir.json)."""
    x = token_embedding(m.w["wte.weight"], ids)
    x = position_embedding(x, m.w["wpe.weight"], 0)
    for layer in range(m.n_layer):
        x = block(m, layer, x, round_to)
    return lm_head(m, x, round_to)


# --------------------------------------------------------------------------- sampling and generation


def argmax_first(row: np.ndarray) -> int:
    """First maximal index (api.cpp:246-248, std::max_element)."""
    return int(np.argmax(row))


def uniform01(seed: int, stream: int, counter: int) -> float:
    """The framework's counter-based uniform in [0,1): splitmix64 over (seed, stream, counter), top
    24 bits.  ember.cpp draws from std::mt19937 (api.h:300), whose stream no other language
    reproduces; the definition here is the framework's own, restated."""
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + stream * 0xBF58476D1CE4E5B9 + counter * 0x94D049BB133111EB + 0x2545F4914F6CDD1D) & mask
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & mask
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & mask
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


def sample(row: np.ndarray, temperature: float, top_k: int, top_p: float, u: float) -> int:
    """ember.cpp's sampler (api.cpp:238-341) with the draw made by inverse CDF from a given
    uniform u: below temperature 0.05 the first maximal index; else p = softmax((l-max)/T);
    candidates ordered by (p, index) descending; the first top_k of them; then the shortest
    prefix whose sum reaches top_p.  ember.cpp draws from that set with std::discrete_distribution;
    the framework draws from the same set, renormalised, by inverse CDF in index order."""
    row = np.asarray(row, dtype=np.float64)
    V = row.shape[0]
    if temperature < 0.05:
        return argmax_first(row)
    top_k = min(top_k, V)
    if top_k <= 0:
        top_k = V
    p = np.exp((row - row.max()) / temperature)
    p = p / p.sum()
    order = sorted(range(V), key=lambda i: (p[i], i), reverse=True)[:top_k]
    keep = []
    cum = 0.0
    for i in order:
        keep.append(i)
        cum += p[i]
        if cum >= top_p:
            break
    total = sum(p[i] for i in keep)
    target = u * total
    acc = 0.0
    for i in sorted(keep):
        acc += p[i]
        if acc > target:
            return i
    return max(keep)


def generate(m: PlainGPT2, prompt, max_new_tokens: int, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
             seed: int = 0, stream: int = 0, stop_ids=(), round_to=None):
    """Prefill, sample, then one token at a time until a stop id, max_new_tokens or the position
    table is full (api.cpp:989-991, 1166-1174, 1355-1356, 1512-1521); every step recomputes the
    whole sequence.  Returns (tokens, finish_reason)."""
    ids = list(prompt)
    out = []
    while True:
        row = forward(m, ids, round_to)[-1]
        tok = sample(row, temperature, top_k, top_p, uniform01(seed, stream, len(out)))
        out.append(tok)
        if tok in stop_ids:
            return out, "stop"
        if len(out) >= max_new_tokens:
            return out, "length"
        if len(ids) + 1 > m.n_positions:  # no position left at which the new token could be fed
            return out, "context"
        ids.append(tok)
