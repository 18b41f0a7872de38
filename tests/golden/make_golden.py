"""Makes tests/golden/*.npz: logits of ember.cpp's own CPU interpreter on tiny random GPT-2 models.

Run by hand where ember.cpp's sources are at hand (they compile on the CPU with g++ alone):

    python tests/golden/make_golden.py --reference /path/to/ember.cpp [--json-include DIR]

For each tiny configuration it writes a model folder with the library's random-weights mode,
converts it to the GGUF that ember.cpp reads (float32 tensors under llama.cpp's GPT-2 names, the
Conv1D matrices transposed to [out, in]), compiles ember.cpp's `tools/ir_logits.cpp` with its
interpreter sources, replays a few id lists (whole prompt and token by token) and stores ids and
logits.  Configuration A runs on the graph that ember.cpp builds itself from the metadata;
configuration B (erf GELU, untied head, attention scale divided by layer + 1) runs on that graph
edited through ember.cpp's EMBER_IR side file: `approx` "none" on the gelu node, and an `affine`
node that multiplies q by 1/(layer+1) before the attention node.  tests/test_plain.py compares
the plain implementation with these files; nothing else reads them.
"""
from __future__ import annotations

import argparse
import json
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

SOURCES = ["graph_ir.cpp", "graph_ir_ops.cpp", "graph_ir_expr.cpp", "graph_ir_mamba.cpp", "graph_ir_recurrence.cpp",
           "graph_ir_validate.cpp", "ir_digest.cpp", "cpu_attention.cpp", "utils.cpp", "logger.cpp", "quantization.cpp",
           "gguf_parser.cpp", "parallel_for.cpp", "model_config.cpp", "weight_management.cpp", "tools/ir_logits.cpp"]

CONFIGS = {
    "tiny_a": dict(vocab_size=512, n_positions=128, n_embd=64, n_layer=2, n_head=4, n_inner=256,
                   activation_function="gelu_new", layer_norm_epsilon=1e-5, tie_word_embeddings=True),
    "tiny_b": dict(vocab_size=1000, n_positions=96, n_embd=96, n_layer=3, n_head=3, n_inner=320,
                   activation_function="gelu", layer_norm_epsilon=1e-6, tie_word_embeddings=False,
                   scale_attn_by_inverse_layer_idx=True),
}
SEEDS = {"tiny_a": 0, "tiny_b": 1}
LENGTHS = (1, 7, 33)


def gguf_bytes(meta: list, tensors: list[tuple[str, np.ndarray]]) -> bytes:
    """GGUF v3 with u32 / f32 / string metadata and float32 tensors (the writer pattern of
    ember.cpp's tools/llama_ir_parity_test.cpp:31-140)."""
    out = bytearray(b"GGUF")
    out += struct.pack("<I", 3) + struct.pack("<Q", len(tensors)) + struct.pack("<Q", len(meta))

    def s(text):
        b = text.encode()
        return struct.pack("<Q", len(b)) + b

    for key, val in meta:
        out += s(key)
        if isinstance(val, str):
            out += struct.pack("<I", 8) + s(val)
        elif isinstance(val, float):
            out += struct.pack("<I", 6) + struct.pack("<f", val)
        else:
            out += struct.pack("<I", 4) + struct.pack("<I", val)
    offset = 0
    offsets = []
    for name, a in tensors:
        out += s(name) + struct.pack("<I", a.ndim)
        for dim in reversed(a.shape):  # ne[0] is the contiguous dimension
            out += struct.pack("<Q", dim)
        out += struct.pack("<I", 0) + struct.pack("<Q", offset)
        offsets.append(offset)
        offset += (a.size * 4 + 31) // 32 * 32
    while len(out) % 32:
        out += b"\0"
    base = len(out)
    out += bytes(offset)
    for (name, a), off in zip(tensors, offsets):
        raw = np.ascontiguousarray(a, dtype="<f4").tobytes()
        out[base + off: base + off + len(raw)] = raw
    return bytes(out)


def to_gguf(plain, path: str) -> None:
    w = plain.w
    f32 = lambda a: np.asarray(a, dtype=np.float32)  # noqa: E731
    tensors = [("token_embd.weight", f32(w["wte.weight"])), ("position_embd.weight", f32(w["wpe.weight"]))]
    for i in range(plain.n_layer):
        p, b = f"h.{i}.", f"blk.{i}."
        tensors += [(b + "attn_norm.weight", f32(w[p + "ln_1.weight"])), (b + "attn_norm.bias", f32(w[p + "ln_1.bias"])),
                    (b + "attn_qkv.weight", f32(w[p + "attn.c_attn.weight"].T)),
                    (b + "attn_qkv.bias", f32(w[p + "attn.c_attn.bias"])),
                    (b + "attn_output.weight", f32(w[p + "attn.c_proj.weight"].T)),
                    (b + "attn_output.bias", f32(w[p + "attn.c_proj.bias"])),
                    (b + "ffn_norm.weight", f32(w[p + "ln_2.weight"])), (b + "ffn_norm.bias", f32(w[p + "ln_2.bias"])),
                    (b + "ffn_up.weight", f32(w[p + "mlp.c_fc.weight"].T)), (b + "ffn_up.bias", f32(w[p + "mlp.c_fc.bias"])),
                    (b + "ffn_down.weight", f32(w[p + "mlp.c_proj.weight"].T)),
                    (b + "ffn_down.bias", f32(w[p + "mlp.c_proj.bias"]))]
    tensors += [("output_norm.weight", f32(w["ln_f.weight"])), ("output_norm.bias", f32(w["ln_f.bias"]))]
    if not plain.tied:
        tensors.append(("output.weight", f32(w["lm_head.weight"])))
    meta = [("general.architecture", "gpt2"), ("general.name", "tiny-gpt2"), ("general.alignment", 32),
            ("gpt2.context_length", plain.n_positions), ("gpt2.embedding_length", plain.n_embd),
            ("gpt2.block_count", plain.n_layer), ("gpt2.feed_forward_length", plain.n_inner),
            ("gpt2.attention.head_count", plain.n_head), ("gpt2.attention.layer_norm_epsilon", float(plain.eps))]
    with open(path, "wb") as f:
        f.write(gguf_bytes(meta, tensors))


def compile_ir_logits(reference: str, json_include: str, build: str) -> str:
    exe = os.path.join(build, "ir_logits")
    cmd = ["g++", "-std=c++17", "-O1", "-fopenmp", "-ffp-contract=off", f"-I{reference}", f"-I{json_include}",
           *[os.path.join(reference, s) for s in SOURCES], "-o", exe]
    print("compiling ember.cpp's interpreter (about a minute) ...", flush=True)
    subprocess.run(cmd, check=True)
    return exe


def find_json_include() -> str:
    import site
    for base in site.getsitepackages():
        cand = os.path.join(base, "include", "cudnn_frontend", "thirdparty")
        if os.path.isfile(os.path.join(cand, "nlohmann", "json.hpp")):
            return cand
    raise SystemExit("nlohmann/json.hpp not found; pass --json-include")


def edit_ir_for_b(ir: dict, n_layer: int) -> dict:
    """erf GELU and q * 1/(layer+1) before the attention node."""
    out = []
    for node in ir["block"]["nodes"]:
        if node.get("op") == "gelu":
            node["approx"] = "none"
        if node.get("op") == "attention":
            out.append({"op": "affine", "in": ["q"], "out": "q",
                        "scale": {"per_layer": [1.0 / (layer + 1) for layer in range(n_layer)]}, "shift": 0.0})
        out.append(node)
    ir["block"]["nodes"] = out
    return ir


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--json-include", default=None)
    args = ap.parse_args()
    import plain_gpt2

    import ember_cpp_b200 as E

    inc = args.json_include or find_json_include()
    with tempfile.TemporaryDirectory() as tmp:
        exe = compile_ir_logits(args.reference, inc, tmp)
        for name, cfgd in CONFIGS.items():
            folder = os.path.join(tmp, name)
            E.write_random_model(folder, E.GPT2Config.from_dict(cfgd), SEEDS[name])
            plain = plain_gpt2.PlainGPT2(folder)
            gguf = os.path.join(tmp, name + ".gguf")
            to_gguf(plain, gguf)
            rng = np.random.default_rng(SEEDS[name] + 100)
            seqs = [rng.integers(0, plain.vocab, n).tolist() for n in LENGTHS]
            env = dict(os.environ, OMP_NUM_THREADS="4")
            if name == "tiny_b":
                printed = os.path.join(tmp, "built.json")
                subprocess.run([exe, gguf], input="[[1]]", text=True, capture_output=True, check=True,
                               env=dict(env, EMBER_IR_PRINT=printed))
                with open(printed) as f:
                    ir = edit_ir_for_b(json.load(f), plain.n_layer)
                side = os.path.join(tmp, "side.json")
                with open(side, "w") as f:
                    json.dump(ir, f)
                env["EMBER_IR"] = side
            r = subprocess.run([exe, gguf], input=json.dumps(seqs), text=True, capture_output=True, env=env)
            if r.returncode != 0:
                print(r.stderr[-3000:])
                raise SystemExit(f"ir_logits failed on {name}")
            recs = json.loads(r.stdout)
            import hashlib
            with open(os.path.join(folder, "model.safetensors"), "rb") as f:
                digest = hashlib.sha256(f.read()).hexdigest()
            save = {"seed": np.int64(SEEDS[name]), "weights_sha256": np.frombuffer(digest.encode(), dtype=np.uint8),
                    "config": np.frombuffer(json.dumps(cfgd).encode(), dtype=np.uint8)}
            for i, (ids, rec) in enumerate(zip(seqs, recs)):
                pre = np.asarray(rec["prefill"], dtype=np.float32)
                dec = np.asarray(rec["decode"], dtype=np.float32)
                print(name, len(ids), "decode rows bit-identical to prefill rows:", bool(np.array_equal(pre, dec)))
                save[f"ids{i}"] = np.asarray(ids, dtype=np.int32)
                save[f"prefill{i}"] = pre
                save[f"decode_equals_prefill{i}"] = np.bool_(np.array_equal(pre, dec))
            np.savez_compressed(os.path.join(HERE, name + ".npz"), **save)
            print("wrote", name + ".npz")
    return 0


if __name__ == "__main__":
    sys.exit(main())
