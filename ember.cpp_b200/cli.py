"""Command line, in the manner of ember.cpp's `tinyllama` (main.cpp:10-39, 121-248).

    ember <model_path> <tokenizer_path> <num_threads> <prompt|batch> [prompt] [options]

The positional arguments and the options keep ember.cpp's names and meanings:
--max-tokens/-mt (256), --n-gpu-layers/-ngl (-1), --use-mmap, --temperature/-t (0.1), --top-k/-k
(40), --top-p/-p (0.9), --use-kv-quant/-kvq, --use-batch-generation/-ubg, --batch-prompts/-bp,
--max-batch-size/-mbs (8).  This library has no tokenizer: a prompt is a string of token ids
("464 3290 318"), the reply is printed as ids, `tokenizer_path` and `num_threads` are accepted
and unused ("-" will do), and `chat` mode, which needs text, is refused.  Options of its own:
--dtype, --seed, --stop, --cache-tokens, and the random-weights mode

    ember <new_model_dir> - 1 random-weights --config config.json --seed 0 [--weights-dtype bfloat16]

which writes config.json and model.safetensors into <new_model_dir>.
"""
from __future__ import annotations

import json
import sys

USAGE = ("Usage: ember <model_path> <tokenizer_path> <num_threads> <prompt|batch|random-weights> [prompt ids] "
         "[--max-tokens N] [--n-gpu-layers -1] [--use-mmap true] [--temperature T] [--top-k K] [--top-p P] "
         "[--use-kv-quant false] [--use-batch-generation true] [--batch-prompts \"ids\" \"ids\" ...] "
         "[--max-batch-size N] [--dtype bfloat16|float32] [--seed S] [--stop \"ids\"] [--cache-tokens N] "
         "[--config FILE] [--weights-dtype bfloat16|float32]")


def parse_ids(text: str) -> list[int]:
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise SystemExit(f"ERROR: a prompt is a list of token ids, got {text!r}") from None


def _flag(value: str, name: str) -> bool:
    v = value.lower()
    if v in ("true", "1"):
        return True
    if v in ("false", "0"):
        return False
    raise SystemExit(f"ERROR: Invalid {name} value: {value}")


def parse_args(argv: list[str]) -> dict:
    if len(argv) >= 1 and argv[0] in ("-h", "--help"):
        print(USAGE)
        print(__doc__)
        raise SystemExit(0)
    if len(argv) < 4:
        print("ERROR: Missing required arguments.", file=sys.stderr)
        print(USAGE, file=sys.stderr)
        raise SystemExit(1)
    a = {"model_path": argv[0], "tokenizer_path": argv[1], "num_threads": argv[2], "mode": argv[3], "prompt": None,
         "max_tokens": 256, "n_gpu_layers": -1, "use_mmap": True, "temperature": 0.1, "top_k": 40, "top_p": 0.9,
         "use_kv_quant": False, "use_batch_generation": False, "batch_prompts": [], "max_batch_size": 8,
         "dtype": "bfloat16", "seed": 0, "stop": None, "cache_tokens": None, "config": None,
         "weights_dtype": "bfloat16"}
    valued = {"--max-tokens": ("max_tokens", int), "-mt": ("max_tokens", int),
              "--n-gpu-layers": ("n_gpu_layers", int), "-ngl": ("n_gpu_layers", int),
              "--temperature": ("temperature", float), "-t": ("temperature", float),
              "--top-k": ("top_k", int), "-k": ("top_k", int), "--top-p": ("top_p", float), "-p": ("top_p", float),
              "--max-batch-size": ("max_batch_size", int), "-mbs": ("max_batch_size", int),
              "--dtype": ("dtype", str), "--seed": ("seed", int), "--stop": ("stop", parse_ids),
              "--cache-tokens": ("cache_tokens", int), "--config": ("config", str),
              "--weights-dtype": ("weights_dtype", str)}
    flags = {"--use-mmap": "use_mmap", "--use-kv-quant": "use_kv_quant", "-kvq": "use_kv_quant",
             "--use-batch-generation": "use_batch_generation", "-ubg": "use_batch_generation"}
    i = 4
    while i < len(argv):
        arg = argv[i]
        if arg in valued or arg in flags:
            if i + 1 >= len(argv):
                raise SystemExit(f"ERROR: {arg} requires a value.")
            if arg in valued:
                key, conv = valued[arg]
                try:
                    a[key] = conv(argv[i + 1])
                except ValueError:
                    raise SystemExit(f"ERROR: Invalid {key}: {argv[i + 1]}") from None
            else:
                a[flags[arg]] = _flag(argv[i + 1], flags[arg])
            i += 2
        elif arg in ("--batch-prompts", "-bp"):
            i += 1
            while i < len(argv) and not argv[i].startswith("-"):
                a["batch_prompts"].append(parse_ids(argv[i]))
                i += 1
            if not a["batch_prompts"]:
                raise SystemExit("ERROR: --batch-prompts requires at least one prompt.")
        elif arg in ("--system-prompt", "-sp", "--rep-penalty", "-rp", "--raw-prompt"):
            raise SystemExit(f"ERROR: {arg} works on text or penalties, which this library does not have.")
        elif a["prompt"] is None and not arg.startswith("-"):
            a["prompt"] = parse_ids(arg)
            i += 1
        elif not arg.startswith("-"):
            raise SystemExit(f"ERROR: Unexpected positional argument: {arg}")
        else:
            raise SystemExit(f"ERROR: Unknown option: {arg}")
    return a


def main(argv: list[str] | None = None) -> int:
    a = parse_args(sys.argv[1:] if argv is None else argv)
    mode = a["mode"]
    if mode == "random-weights":
        import torch

        from .config.base import config_from_dict
        from .weights.random_init import write_random_model
        if not a["config"]:
            raise SystemExit("ERROR: random-weights needs --config FILE (a config.json).")
        with open(a["config"]) as f:
            cfg = config_from_dict(json.load(f))
        dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}.get(a["weights_dtype"])
        if dt is None:
            raise SystemExit(f"ERROR: Invalid weights_dtype: {a['weights_dtype']}")
        print(write_random_model(a["model_path"], cfg, a["seed"], dt))
        return 0
    if mode == "chat":
        raise SystemExit("ERROR: chat mode needs a tokenizer; this library works on token ids (use prompt or batch).")
    if mode not in ("prompt", "batch"):
        print(f"ERROR: Invalid mode '{mode}'. Expected 'prompt' or 'batch'.", file=sys.stderr)
        print(USAGE, file=sys.stderr)
        return 1
    if mode == "batch":
        if not a["batch_prompts"]:
            raise SystemExit('ERROR: Batch mode requires prompts. Use --batch-prompts "ids" "ids" ...')
        if len(a["batch_prompts"]) > a["max_batch_size"]:
            raise SystemExit(f"ERROR: Number of prompts ({len(a['batch_prompts'])}) exceeds max batch size "
                             f"({a['max_batch_size']})")
    elif a["prompt"] is None:
        raise SystemExit("ERROR: prompt mode needs a prompt: a quoted list of token ids.")

    from .api import Session
    try:
        session = Session(a["model_path"], a["tokenizer_path"], 1, a["n_gpu_layers"], a["use_mmap"], a["use_kv_quant"],
                          True if mode == "batch" else a["use_batch_generation"],
                          a["max_batch_size"] if mode == "batch" else 1, dtype=a["dtype"],
                          max_tokens=a["cache_tokens"], seed=a["seed"])
        prompts = a["batch_prompts"] if mode == "batch" else [a["prompt"]]
        results = session.generate_detailed(prompts, a["max_tokens"], a["temperature"], a["top_k"], a["top_p"], a["stop"])
    except (ValueError, RuntimeError, OSError) as e:
        print(f"Error: {e}", file=sys.stderr)
        return 1
    if mode == "prompt":
        print(" ".join(str(t) for t in results[0].tokens))
    else:
        print("=" * 80)
        print("BATCH PROCESSING RESULTS")
        print("=" * 80)
        for n, (p, r) in enumerate(zip(prompts, results), 1):
            print(f"\n--- Prompt {n} ---")
            print("Input: " + " ".join(str(t) for t in p))
            print("Output: " + " ".join(str(t) for t in r.tokens) + f"   [{r.finish_reason}]")
    return 0


if __name__ == "__main__":
    sys.exit(main())
