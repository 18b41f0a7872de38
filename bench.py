"""Benchmark of the library on one B200: decode tokens per second of GPT-2 XL shape with random
weights (batch 8 by default, 128-token prompts decoded towards the 1,024-token context), with the
2,048-token prefill, the decode step's memory roofline and batch 1 / 64 beside it.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch B] [--impl ours|reference]
    python bench.py --linear M N K [--act gelu_tanh] [--residual]      (one product, every kernel that takes it)

Prints ONE JSON line on stdout (everything else goes to stderr).  A "step" is one decode step of
the whole batch.  `value` times K steps of the engine's own loop (step function + device sampler,
every step's ids read back to the host; the loop, like the library's generation loop, queues a step
with the ids of the step before still on the device and reads them afterwards) with CUDA events; `e2e` is the same count of tokens through the Python
entry point (`Session.generate_batch`, host ids in, host ids out) by wall clock between its first
and last new token.  ember.cpp publishes no GPT-2 speed, so `vs_baseline` is null.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

XL = dict(vocab_size=50257, n_positions=1024, n_embd=1600, n_layer=48, n_head=25, n_inner=6400,
          activation_function="gelu_new", layer_norm_epsilon=1e-5, tie_word_embeddings=True)
PROMPT_LEN = 128
PREFILL = (2, 1024)


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def xl_config() -> dict:
    """The sizes of BASELINE.json's configs[2] (read from the file when it is there)."""
    cfg = dict(XL)
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            text = json.load(f)["configs"][2]
        for key in ("n_layer", "n_embd", "n_head", "n_inner", "n_positions"):
            m = re.search(key + r"=(\d+)", text)
            if m:
                cfg[key] = int(m.group(1))
        m = re.search(r"vocab=(\d+)", text)
        if m:
            cfg["vocab_size"] = int(m.group(1))
    except (OSError, KeyError, IndexError, ValueError):
        pass
    return cfg


def peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed regions run (read only)."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows) -> dict:
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        sm, mx, reasons = [], [], set()
        for t, cols in self.rows:
            if len(cols) < 6 or not any(a <= t <= b for a, b in windows):
                continue
            try:
                sm.append(float(cols[0]))
                mx.append(float(cols[1]))
            except ValueError:
                continue
            for name, v in zip(names, cols[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args) -> int:
    """ember.cpp's own GPT-2 path (its graph interpreter on its CUDA path, float32, unmodified) on the
    same model shape and workload, through baseline/_ref/ref_bench.  The package does not install with
    pip offline (its CMake configure downloads two libraries); its interpreter is built by hand from its
    sources instead (baseline/build_reference.py), where those sources are mounted."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import build_reference
    import reference_arm as arm
    exe = build_reference.binary()
    if not os.path.isfile(exe):
        src = os.environ.get("EMBER_REFERENCE", "/root/reference")
        try:
            exe = build_reference.build(src)
        except (RuntimeError, OSError) as e:
            why = " ".join(str(e).split())[:300]
            print(json.dumps({"impl": "reference", "unavailable": f"baseline/_ref/ref_bench is not built and cannot be built here: {why}"}))
            return 0
    cfg = dict(xl_config())
    if args.layers:
        cfg["n_layer"] = args.layers
    W = max(3, args.warmup)
    K = args.steps if args.steps is not None else cfg["n_positions"] - args.prompt_len - W
    K = max(1, min(K, cfg["n_positions"] - args.prompt_len - W))
    clocks = ClockSampler()
    clocks.start()
    t0 = time.time()
    try:
        line = arm.run(exe, cfg, args.batch, args.prompt_len, W, K, PREFILL)
    except (RuntimeError, OSError, subprocess.SubprocessError, ValueError) as e:
        clocks.stop()
        print(json.dumps({"impl": "reference", "unavailable": " ".join(str(e).split())[:300]}))
        return 0
    clocks.stop()
    line["clocks"] = clocks.summary([(t0, time.time())])
    print(json.dumps(line))
    return 0


def linear_mode(args) -> int:
    """Times one bfloat16 product Y[M,N] = X[M,K] W[N,K]^T (+ bias, activation, float32 residual) on every
    kernel that takes its shape: cuBLASLt (`lt`), this library's tcgen05 kernel (`tc`, more than 64 rows), the
    tcgen05 weight-streaming kernel (`stream`, up to 64 rows) and the mma.sync weight-streaming kernel
    (`decode`, up to 16 rows).  As in a model's step, the launches follow one another in a captured graph,
    each with a weight matrix of its own (so many that they exceed L2 together: weights come from DRAM
    every time); the time is the graph's CUDA-event time divided by its launches, the median of 7 replays."""
    import torch

    from ember_cpp_b200.csrc.ops import CudaOps
    M, N, K = args.linear
    ops = CudaOps()
    copies = max(4, -(-(400 << 20) // (N * K * 2)))
    x = torch.randn(M, K, device="cuda").bfloat16()
    ws = [(torch.randn(N, K, device="cuda") * 0.02).bfloat16() for _ in range(copies)]
    bias = torch.randn(N, device="cuda")
    res = torch.randn(M, N, device="cuda") if args.residual else None
    out = res if res is not None else torch.empty(M, N, device="cuda", dtype=torch.bfloat16)

    def timed(fn):
        for w in ws[:2]:
            fn(w)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for w in ws:
                fn(w)
        graph.replay()
        times = []
        for _ in range(7):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3 / len(ws))
        ops.check()
        return statistics.median(times)

    def lt(w):
        ops.gemm, ops.linear_stream_on = "lt", False
        ops.linear(x, w, bias, act=args.act, residual=res, out_dtype=out.dtype)

    kernels = {}
    if M > 16:
        kernels["lt"] = lt
    if M > 64:
        kernels["tc"] = lambda w: ops.linear_tc(x, w, bias, args.act, res, out)
    if M <= 64:
        kernels["stream"] = lambda w: ops.linear_stream(x, w, bias, args.act, res, out)
    if M <= 16:
        def decode(w):
            ops.linear_stream_on = False
            ops.linear(x, w, bias, act=args.act, residual=res, out_dtype=out.dtype)
        kernels["decode"] = decode
    ideal = N * K * 2 / (peaks()["hbm_gbs"] * 1e3)
    for name, fn in kernels.items():
        us = timed(fn)
        print(f"{name:7s} M={M} N={N} K={K} act={args.act} residual={args.residual}: {us:7.1f} us a launch, "
              f"{2.0 * M * N * K / us / 1e6:7.1f} TFLOP/s, weights at {N * K * 2 / us / 1e3:6.0f} GB/s "
              f"(streaming W alone: {ideal:.1f} us)")
    return 0


def umma_issue_mode() -> int:
    """Cycles per tcgen05.mma by shape and by the way it is issued (see csrc/umma_probe.cu)."""
    from ember_cpp_b200.csrc.ops import CudaOps
    ops = CudaOps()
    for m in (128, 64):
        for n in (16, 64, 128, 256):
            for elected in (False, True):
                ops.umma_issue_probe(m, n, 64, elected)
                issue, done = ops.umma_issue_probe(m, n, 512, elected)
                print(f"M={m:3d} N={n:3d} {'elect.sync, whole warp ' if elected else 'if (thread == 0)       '}: {issue:6.1f} cycles to issue, "
                      f"{done:6.1f} until complete, {2.0 * m * n * 16 / done:6.0f} flop a cycle")
    for every in (1, 4, 8, 16):
        for wait_too in (False, True):
            issue, done = ops.umma_issue_probe(128, 64, 512, True, commit_every=every, wait_too=wait_too)
            print(f"M=128 N= 64 elect.sync, a tcgen05.commit after every {every:2d}{', a satisfied wait and a fence before' if wait_too else ''}: "
                  f"{issue * every:6.1f} cycles a group, {issue:6.1f} a product")
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="tokens of each prompt before decoding starts")
    ap.add_argument("--only", default=None, choices=["prefill"],
                    help="run only the 2,048-token prefill (a few repeats; prints its line and no benchmark record): for profiling")
    ap.add_argument("--kernels", action="store_true",
                    help="with --only prefill: one more step under torch's profiler, and the device time of each of its kernels")
    ap.add_argument("--linear", type=int, nargs=3, metavar=("M", "N", "K"), default=None,
                    help="time one bfloat16 product on every kernel that takes it, instead of the benchmark")
    ap.add_argument("--act", default=None, choices=[None, "gelu_tanh", "gelu_erf"], help="with --linear: the epilogue's activation")
    ap.add_argument("--residual", action="store_true", help="with --linear: add a float32 residual (the output is float32 then)")
    ap.add_argument("--umma-issue", action="store_true", help="print what a tcgen05.mma costs to issue, by shape and way of issuing")
    args = ap.parse_args()
    if args.umma_issue:
        return umma_issue_mode()
    if args.linear:
        return linear_mode(args)
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library runs a model on a single GPU (asked for {args.gpus})")
        return 2

    import numpy as np
    import torch

    import ember_cpp_b200 as E
    from ember_cpp_b200.config import get_architecture
    from ember_cpp_b200.engine import Engine
    from ember_cpp_b200.parts import DecoderModel
    from ember_cpp_b200.weights import random_tensors

    W = max(3, args.warmup)
    prompt_len = args.prompt_len
    cfgd = xl_config()
    full_layers = cfgd["n_layer"]
    if args.layers:
        cfgd["n_layer"] = args.layers
    cfg = E.GPT2Config.from_dict({**cfgd, "architectures": ["GPT2LMHeadModel"]})
    ctx = cfg.n_positions
    K = args.steps if args.steps is not None else ctx - prompt_len - W
    K = max(1, min(K, ctx - prompt_len - W))
    pk = peaks()

    def build_engine(config, max_tokens):
        t0 = time.time()
        spec = get_architecture(config.architecture).build_spec(config)
        tensors = random_tensors(DecoderModel(spec).weight_specs(), seed=0, dtype=torch.bfloat16, device="cuda")
        log(f"random weights: {sum(t.numel() for t in tensors.values()) / 1e9:.3f} G parameters in {time.time() - t0:.1f} s")
        eng = Engine.from_spec(spec, tensors, dtype="bfloat16", max_tokens=max_tokens)
        eng.config = config
        return eng

    def step_bytes(config):
        """(bytes of weights a decode step reads once, bytes of cache per held position)."""
        d, L, F, V = config.n_embd, config.n_layer, config.inner, config.vocab_size
        weights = L * (3 * d * d + d * d + 2 * d * F) * 2 + V * d * 2 + L * (3 * d + d + F + d + 4 * d) * 4 + 2 * d * 4
        return weights, L * 2 * d * 2

    biggest = max(args.batch, 1 if args.no_points else 64)
    engine = build_engine(cfg, max(biggest, PREFILL[0]) * ctx)
    sampler = E.Sampler(engine.ops)
    params = E.SamplingParams()  # ember.cpp's defaults: temperature 0.1, top_k 40, top_p 0.9
    rng = np.random.default_rng(0)
    d, L, F, V = cfg.n_embd, cfg.n_layer, cfg.inner, cfg.vocab_size
    clocks = ClockSampler()
    clocks.start()
    windows = []

    def decode_run(eng, lengths, warm: int, steps: int | None):
        """Prefills prompts of the given lengths in one step, then decodes: `warm` untimed steps and then `steps`
        timed ones, or (steps None) until every sequence has reached the context's end, sequences leaving as
        they do.  As Generator does, a step takes its tokens from the sampler's output on the device and is
        queued before the host reads those ids."""
        config = eng.config
        weight_bytes, kv_bytes_per_pos = step_bytes(config)
        smp = sampler if eng is engine else E.Sampler(eng.ops)
        B = len(lengths)
        # the step's graphs for every bucket of lengths (and, where the batch shrinks, of batch sizes), before anything is timed
        for b in ([B] if steps is not None else [1 << k for k in range(B.bit_length()) if (1 << k) <= B] + [B]):
            eng.capture_decode(b)
        slots = [eng.open() for _ in range(B)]
        prompts = [rng.integers(0, config.vocab_size, n).tolist() for n in lengths]
        logits = eng.step([(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        ids = smp.sample(logits, params, list(range(B)), [0] * B, out=eng.sample_target(B))
        on_the_way = smp.fetch(ids)
        live = list(range(B))
        rows = list(range(B))
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        cache_bytes = tokens = timed_steps = launches0 = 0
        i = 0
        w0 = time.time()
        while live and (steps is None or i < warm + steps):
            if i == warm:
                torch.cuda.synchronize()
                launches0 = eng.ops.launches
                w0 = time.time()
                start.record()
            if i >= warm:
                cache_bytes += sum(eng.length(slots[j]) + 1 for j in live) * kv_bytes_per_pos
                tokens += len(live)
                timed_steps += 1
            logits = eng.step([(slots[j], [0], [0]) for j in live], borrow=True, device_tokens=(ids, rows))
            following = smp.sample(logits, params, live, [i + 1] * len(live), out=eng.sample_target(len(live)))
            fetched = smp.fetch(following)
            on_the_way.tolist()
            ids, on_the_way = following, fetched
            i += 1
            if steps is None:      # sequences that have reached the context's end leave; the others keep their rows' order
                staying = [k for k, j in enumerate(live) if eng.length(slots[j]) < config.n_positions]
                for k, j in enumerate(live):
                    if k not in staying:
                        eng.close(slots[j])
                live = [live[k] for k in staying]
                rows = staying
            else:
                rows = list(range(len(live)))
        on_the_way.tolist()
        stop.record()
        torch.cuda.synchronize()
        windows.append((w0, time.time()))
        ms = start.elapsed_time(stop)
        launches = eng.ops.launches - launches0
        for j in live:
            eng.close(slots[j])
        per_step = weight_bytes + cache_bytes / max(1, timed_steps)
        gbs = per_step / (ms / max(1, timed_steps) / 1e3) / 1e9
        return {"tok_s": tokens / (ms / 1e3), "ms_per_step": ms / max(1, timed_steps), "launches": launches, "steps": timed_steps,
                "bytes_per_step": per_step, "gbs": gbs, "frac": gbs / pk["hbm_gbs"]}

    def roof(r):
        return {"bytes_per_step": int(r["bytes_per_step"]), "gbs": round(r["gbs"], 1), "frac": round(r["frac"], 4),
                "ms_per_step": round(r["ms_per_step"], 4)}

    points, point_roofs = {}, {}
    if args.only != "prefill":
        log("main decode run ...")
        main_run = decode_run(engine, [prompt_len] * args.batch, W, K)
        log(main_run)
        # (right after the run it is compared with: the sweeps below heat the chip into its power cap)
        # the same decode through the Python entry point: host ids in, host ids out
        session = E.Session.from_engine(engine, max_batch_size=args.batch, seed=0)
        stamps = []
        session.set_token_callback(lambda i, tok: stamps.append(time.perf_counter()) if i == 0 else None)
        prompts = [rng.integers(0, V, prompt_len).tolist() for _ in range(args.batch)]
        w0 = time.time()
        out = session.generate_batch(prompts, steps=W + K + 1, temperature=params.temperature, top_k=params.top_k,
                                     top_p=params.top_p, stop_token_ids=[])
        windows.append((w0, time.time()))
        e2e_tok_s = args.batch * K / (stamps[-1] - stamps[-1 - K])
        assert all(len(o) == W + K + 1 for o in out)
        from ember_cpp_b200.engine import StepLayout
        bucket = 1 << (args.batch - 1).bit_length()
        h2d = StepLayout(bucket, bucket, bucket, engine.cache.max_blocks, len(engine.cache.groups)).size * 4

    if not args.no_points and args.only != "prefill":
        for B in (1, 8, 64):       # the whole sweep from the prompt to the context's end, whatever --steps says
            r = decode_run(engine, [PROMPT_LEN] * B, W, ctx - PROMPT_LEN - W)
            points[f"decode_b{B}"] = round(r["tok_s"], 1)
            point_roofs[f"decode_b{B}"] = roof(r)
            log(f"batch {B}: {r}")

    # prefill of 2,048 tokens: 2 prompts x 1,024, the last row's logits wanted
    n_seq, plen = PREFILL
    plen = min(plen, ctx)
    T = n_seq * plen
    times, host_times = [], []
    for rep in range(2 + 5):
        slots = [engine.open() for _ in range(n_seq)]
        prompts = [rng.integers(0, V, plen).tolist() for _ in range(n_seq)]
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.time()
        a.record()
        engine.step([(s, p, [plen - 1]) for s, p in zip(slots, prompts)])
        b.record()
        queued = time.time() - w0          # what the host took to queue the step's launches
        torch.cuda.synchronize()
        if rep >= 2:
            times.append(a.elapsed_time(b))
            host_times.append(queued * 1e3)
            windows.append((w0, time.time()))
        for s in slots:
            engine.close(s)
    pre_ms = statistics.median(times)
    pre_flops = 2 * T * L * (3 * d * d + d * d + 2 * d * F) + n_seq * 2 * d * plen * (plen + 1) * L + 2 * n_seq * d * V
    prefill = {"value": round(T / (pre_ms / 1e3), 1), "tokens": T, "ms": round(pre_ms, 3),
               "frac": round(pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

    if args.only == "prefill":
        clocks.stop()
        line = {"prefill": prefill, "n_layer": L, "times_ms": [round(t, 3) for t in times],
                "host_queue_ms": [round(t, 3) for t in host_times]}
        if engine.ops.op_timing:     # EMBER_OP_TIMING=1: the time per kernel entry point over the repeats (launches do not overlap then)
            line["op_ms_per_prefill"] = {k: round(ms / len(times + [0, 0]), 4) for k, (n, ms) in sorted(engine.ops.op_times().items())}
        if args.kernels:   # one more step, under torch's profiler (CUPTI): what each kernel takes inside the step
            from torch.profiler import ProfilerActivity, profile
            slots = [engine.open() for _ in range(n_seq)]
            prompts = [rng.integers(0, V, plen).tolist() for _ in range(n_seq)]
            torch.cuda.synchronize()
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                engine.step([(s, p, [plen - 1]) for s, p in zip(slots, prompts)])
                torch.cuda.synchronize()
            for s in slots:
                engine.close(s)
            evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                         key=lambda e: e.time_range.start)
            agg: dict = {}
            for e in evs:
                n, us = agg.get(e.name, (0, 0.0))
                agg[e.name] = (n + 1, us + e.time_range.end - e.time_range.start)
            span = evs[-1].time_range.end - evs[0].time_range.start if evs else 0.0
            line["kernels_us"] = {"span": round(span, 1), "sum": round(sum(us for _, us in agg.values()), 1),
                                  "by_kernel": [[name[:64], n, round(us, 1)] for name, (n, us) in
                                                sorted(agg.items(), key=lambda kv: -kv[1][1])[:14]]}
        print(json.dumps(line))
        return 0

    # BASELINE.json's two other workloads at their full depth: GPT-2 large's shape (16 ragged prompts of 1 to 512
    # tokens, then 256 decode steps) and GPT-2 medium's (64 ragged prompts of 8 to 960 tokens, each decoded to the
    # context's end; sequences leave as they get there)
    if not args.no_points:
        del session
        engine = sampler = None
        torch.cuda.empty_cache()
        for name, sizes, lengths, steps in (
                ("large_b16", dict(n_layer=36, n_embd=1280, n_head=20, n_inner=5120), rng.integers(1, 513, 16).tolist(), 256),
                ("medium_b64", dict(n_layer=24, n_embd=1024, n_head=16, n_inner=4096), rng.integers(8, 961, 64).tolist(), None)):
            c = E.GPT2Config.from_dict({**XL, **sizes, "architectures": ["GPT2LMHeadModel"]})
            eng = build_engine(c, len(lengths) * c.n_positions)
            r = decode_run(eng, [int(n) for n in lengths], W if steps else 0, steps)
            points[name] = round(r["tok_s"], 1)
            point_roofs[name] = roof(r)
            log(f"{name}: {r}")
            del eng
            torch.cuda.empty_cache()
    clocks.stop()

    achieved = main_run["bytes_per_step"] / (main_run["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": "decode tok/s (GPT-2 XL shape, random weights)", "value": round(main_run["tok_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": "gpt2-xl-shape", "n_layer": L, "n_layer_of_config": full_layers, "n_embd": d,
                   "n_head": cfg.n_head, "n_inner": F, "vocab_size": V, "n_positions": ctx, "global_batch": args.batch,
                   "seq_len": ctx, "prompt_len": prompt_len, "context_end": prompt_len + W + K + 1,
                   "parallelism": "single-gpu", "weights": "random seed 0 bf16", "sampling": "t0.1 k40 p0.9",
                   "l2": "inputs>L2 (3.1 GB of weights per step)", "peaks": pk["source"]},
        "e2e": {"value": round(e2e_tok_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": args.batch * 4},
        "gpu_launches": main_run["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "points_roofline": point_roofs,
        "clocks": clocks.summary(windows),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
