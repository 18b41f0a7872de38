"""Timeline of one decode step, launch by launch.

    EMBER_TIMELINE=1 python -m ember_cpp_b200.csrc.timeline [--layers 4] [--batch 8] [--context 576] [--blocks KERNEL] [--steps 1]

builds (once) the instrumented library, runs a model of GPT-2 XL's layer sizes with random weights
for a few one-token steps as a replayed graph, and prints for every launch of the last step when
its first and last block started, passed the wait for the kernel in front, and ended (microseconds
from the step's first mark), on how many SMs its blocks ran and the most that one SM took, with the marks that the kernel's source places in between (A, B, C,
D).  `--blocks attention_decode` adds every block of that kernel's third launch; `--steps 3` reports the
last three steps one after another, which shows what lies between the end of one step and the start of the next.  The instrumented
kernels are a little slower (a mark costs a block's first thread a global timer read and a store).
"""
from __future__ import annotations

import argparse
import os
import sys

NAMES = {0: "start", 1: "dep", 7: "D", 4: "A", 5: "B", 6: "C", 2: "end", 3: "merged"}
ORDER = (0, 1, 7, 4, 5, 6, 2, 3)


def launches_of(marks):
    """Groups (t, kernel, mark, block, grid, sm) into launches: a block's start mark joins the open launch
    of its (kernel, grid) until that launch has all its blocks (or, for a kernel whose idle blocks leave
    no mark, until the block index repeats); its later marks go where its start went."""
    launches, open_, of_block = [], {}, {}
    for t, k, m, b, g, sm in marks:
        key = (k, g)
        if m == 0:
            cur = open_.get(key)
            if cur is None or cur["n"] >= g or b in cur["blocks"]:
                cur = dict(kernel=k, grid=g, n=0, t={}, blocks={}, sms={})
                launches.append(cur)
                open_[key] = cur
            cur["n"] += 1
            cur["sms"][sm] = cur["sms"].get(sm, 0) + 1
            of_block[(k, g, b)] = cur
        cur = of_block.get((k, g, b))
        if cur is None:
            continue
        lo, hi = cur["t"].get(m, (t, t))
        cur["t"][m] = (min(lo, t), max(hi, t))
        cur["blocks"].setdefault(b, {})[m] = t
    launches.sort(key=lambda x: x["t"][0][0])
    return launches


def report(launches, blocks_of: str | None = None) -> str:
    t0 = launches[0]["t"][0][0]
    lines = []
    for cur in launches:
        parts = [f'{cur["kernel"]:17s} grid {cur["grid"]:5d} n {cur["n"]:5d} on {len(cur["sms"]):3d} SMs (<= {max(cur["sms"].values()):2d})']
        for m in ORDER:
            if m in cur["t"]:
                lo, hi = cur["t"][m]
                parts.append(f"{NAMES[m]} {(lo - t0) / 1000:7.2f}..{(hi - t0) / 1000:7.2f}")
        lines.append(" | ".join(parts))
    if blocks_of:
        some = [x for x in launches if x["kernel"] == blocks_of]
        if some:
            cur = some[min(2, len(some) - 1)]
            base = cur["t"][0][0]
            lines.append("")
            for b, marks in sorted(cur["blocks"].items(), key=lambda kv: kv[1].get(0, 0)):
                lines.append(f"block {b:5d} " + " ".join(f"{NAMES[m]} {(marks[m] - base) / 1000:6.2f}" for m in ORDER if m in marks))
    return "\n".join(lines)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=576)
    ap.add_argument("--blocks", default=None, help="a kernel's name: list every block of its third launch")
    ap.add_argument("--steps", type=int, default=1, help="consecutive steps to report (more than one shows the edge between steps)")
    args = ap.parse_args()
    if os.environ.get("EMBER_TIMELINE") != "1":
        print("set EMBER_TIMELINE=1: the marks are compiled in only then", file=sys.stderr)
        return 2
    import numpy as np
    import torch

    from .. import GPT2Config, Sampler, SamplingParams
    from ..config import get_architecture
    from ..engine import Engine
    from ..parts import DecoderModel
    from ..weights import random_tensors

    cfg = GPT2Config.from_dict(dict(architectures=["GPT2LMHeadModel"], vocab_size=50257, n_positions=1024, n_embd=1600,
                                    n_layer=args.layers, n_head=25, n_inner=6400, activation_function="gelu_new",
                                    layer_norm_epsilon=1e-5))
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    tensors = random_tensors(DecoderModel(spec).weight_specs(), seed=0, dtype=torch.bfloat16, device="cuda")
    engine = Engine.from_spec(spec, tensors, dtype="bfloat16", max_tokens=args.batch * cfg.n_positions)
    sampler, params = Sampler(engine.ops), SamplingParams()
    rng = np.random.default_rng(0)
    slots = [engine.open() for _ in range(args.batch)]
    prompts = [rng.integers(0, cfg.vocab_size, args.context).tolist() for _ in range(args.batch)]
    logits = engine.step([(s, p, [args.context - 1]) for s, p in zip(slots, prompts)])
    streams = list(range(args.batch))
    ids = sampler.sample(logits, params, streams, [0] * args.batch, out=engine.sample_target(args.batch))
    rows = list(range(args.batch))
    for i in range(12):
        if i == 12 - max(1, args.steps):  # the last step alone (or the last few)
            torch.cuda.synchronize()
            engine.ops.timeline()
        logits = engine.step([(s, [0], [0]) for s in slots], borrow=True, device_tokens=(ids, rows))
        ids = sampler.sample(logits, params, streams, [i + 1] * args.batch, out=engine.sample_target(args.batch))
    torch.cuda.synchronize()
    print(report(launches_of(engine.ops.timeline()), args.blocks))
    return 0


if __name__ == "__main__":
    sys.exit(main())
