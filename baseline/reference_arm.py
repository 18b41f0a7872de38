"""The reference arm of bench.py: ember.cpp's own GPT-2 path, unmodified, timed on the benchmark's
model shape with random weights.

ember.cpp runs GPT-2 through its graph interpreter from a GGUF file in float32
(graph_ir.cpp:721-766; graph_ir.h:64-66).  This module writes such a file for the benchmark's
configuration (the tensor names and metadata keys that its graph builder reads,
graph_ir.cpp:561-581, 725-729; float32 tensors, ne0 = the input width; the writer pattern of its
tools/llama_ir_parity_test.cpp:31-140), with weights drawn as the benchmark draws them, and runs
`baseline/_ref/ref_bench` on it (built by baseline/build_reference.py from the reference's sources
and baseline/ref_bench.cpp).  Nothing of this repository's engine, models or kernels is on that
path; torch only draws the random numbers.
"""
from __future__ import annotations

import json
import math
import os
import struct
import subprocess
import tempfile


def _s(text: str) -> bytes:
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def tensor_table(cfg: dict) -> list[tuple[str, tuple[int, ...], float, float]]:
    """(name, shape [out, in] or [n], mean, std) of every tensor of a GPT-2 GGUF, in file order."""
    d, F, L = cfg["n_embd"], cfg["n_inner"], cfg["n_layer"]
    proj = 0.02 / math.sqrt(2 * L)
    t = [("token_embd.weight", (cfg["vocab_size"], d), 0.0, 0.02), ("position_embd.weight", (cfg["n_positions"], d), 0.0, 0.02)]
    for i in range(L):
        b = f"blk.{i}."
        t += [(b + "attn_norm.weight", (d,), 1.0, 0.02), (b + "attn_norm.bias", (d,), 0.0, 0.02),
              (b + "attn_qkv.weight", (3 * d, d), 0.0, 0.02), (b + "attn_qkv.bias", (3 * d,), 0.0, 0.01),
              (b + "attn_output.weight", (d, d), 0.0, proj), (b + "attn_output.bias", (d,), 0.0, 0.01),
              (b + "ffn_norm.weight", (d,), 1.0, 0.02), (b + "ffn_norm.bias", (d,), 0.0, 0.02),
              (b + "ffn_up.weight", (F, d), 0.0, 0.02), (b + "ffn_up.bias", (F,), 0.0, 0.01),
              (b + "ffn_down.weight", (d, F), 0.0, proj), (b + "ffn_down.bias", (d,), 0.0, 0.01)]
    t += [("output_norm.weight", (d,), 1.0, 0.02), ("output_norm.bias", (d,), 0.0, 0.02)]
    return t                      # tied head: no output.weight


def write_gguf(path: str, cfg: dict, seed: int = 0) -> int:
    """A GGUF v3 file of float32 tensors for the configuration; returns its size in bytes.  Tensors are
    drawn and written one at a time (the XL shape is 6.2 GB)."""
    import torch
    meta = [("general.architecture", "gpt2"), ("general.name", "bench-gpt2"), ("general.alignment", 32),
            ("gpt2.context_length", cfg["n_positions"]), ("gpt2.embedding_length", cfg["n_embd"]),
            ("gpt2.block_count", cfg["n_layer"]), ("gpt2.feed_forward_length", cfg["n_inner"]),
            ("gpt2.attention.head_count", cfg["n_head"]), ("gpt2.attention.layer_norm_epsilon", float(cfg["layer_norm_epsilon"]))]
    table = tensor_table(cfg)
    head = bytearray(b"GGUF") + struct.pack("<I", 3) + struct.pack("<Q", len(table)) + struct.pack("<Q", len(meta))
    for key, val in meta:
        head += _s(key)
        if isinstance(val, str):
            head += struct.pack("<I", 8) + _s(val)
        elif isinstance(val, float):
            head += struct.pack("<I", 6) + struct.pack("<f", val)
        else:
            head += struct.pack("<I", 4) + struct.pack("<I", val)
    offset = 0
    for name, shape, _, _ in table:
        head += _s(name) + struct.pack("<I", len(shape))
        for dim in reversed(shape):          # ne[0] is the contiguous dimension
            head += struct.pack("<Q", dim)
        head += struct.pack("<I", 0) + struct.pack("<Q", offset)     # type 0: F32
        n = 4 * math.prod(shape)
        offset += (n + 31) // 32 * 32
    head += b"\0" * (-len(head) % 32)
    device = "cuda" if torch.cuda.is_available() else "cpu"
    gen = torch.Generator(device=device).manual_seed(seed)
    with open(path, "wb") as f:
        f.write(head)
        for name, shape, mean, std in table:
            a = torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std + mean
            raw = a.cpu().numpy().tobytes()
            f.write(raw)
            f.write(b"\0" * (-len(raw) % 32))
    return os.path.getsize(path)


def run(binary: str, cfg: dict, batch: int, prompt_len: int, warmup: int, steps: int, prefill=(2, 1024), seed: int = 0) -> dict:
    """Writes the model, runs ember.cpp's interpreter on it and returns bench.py's JSON line as a dict."""
    with tempfile.TemporaryDirectory() as tmp:
        gguf = os.path.join(tmp, "model.gguf")
        size = write_gguf(gguf, cfg, seed)
        n_seq, plen = prefill
        plen = min(plen, cfg["n_positions"])
        env = dict(os.environ, OMP_NUM_THREADS="8")
        r = subprocess.run([binary, gguf, str(prompt_len), str(warmup), str(steps), str(n_seq * plen), str(n_seq)],
                           capture_output=True, text=True, cwd=tmp, env=env, timeout=1500)
    if r.returncode != 0:
        raise RuntimeError(f"ref_bench exited {r.returncode}: {r.stderr.strip()[-400:]}")
    m = json.loads(r.stdout.strip().splitlines()[-1])
    tok_s = 1e3 / m["decode_ms_per_step"]
    V = cfg["vocab_size"]
    return {
        "metric": "decode tok/s (GPT-2 XL shape, random weights)", "value": round(tok_s, 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": m["steps"], "warmup": m["warmup"], "ms_per_step": round(m["decode_ms_per_step"] * batch, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "impl": "reference",
        "config": {"model": "gpt2-xl-shape", "n_layer": cfg["n_layer"], "n_layer_of_config": cfg["n_layer"],
                   "n_embd": cfg["n_embd"], "n_head": cfg["n_head"], "n_inner": cfg["n_inner"], "vocab_size": V,
                   "n_positions": cfg["n_positions"], "global_batch": batch, "seq_len": cfg["n_positions"],
                   "prompt_len": prompt_len, "context_end": m["context_end"], "parallelism": "single-gpu",
                   "weights": f"random seed {seed} fp32 gguf ({size / 1e9:.1f} GB)", "sampling": "argmax on the host",
                   "batching": "one sequence at a time (Interpreter::forward holds one): a batch's rate is one sequence's",
                   "timer": "wall clock around synchronous forward calls", "path": "ember_ir::Interpreter, device path",
                   "kv": m["kv_format"]},
        "e2e": {"value": round(tok_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4 * V},
        "gpu_launches": None,
        "prefill": {"value": round(m["prefill_tokens"] / (m["prefill_ms"] / 1e3), 1), "tokens": m["prefill_tokens"],
                    "ms": round(m["prefill_ms"], 3)},
    }
