"""Command line: ``python -m transformer_b200 <verb> ...``

The reference has no command line; its driver is a test configured by environment variables
(test-utils/src/lib.rs:31-84, docs/user-guide/doc.md:150-159).  The options here carry those
names and meanings, and each falls back to the variable of the same name:

    --model        TEST_MODEL    model folder (config.json + model.safetensors); required
    --devices      DEVICES       GPU index, default 0 (models/llama/cuda/src/infer.rs:47)
    --prompt       PROMPT        the prompt; token ids separated by commas or blanks (no tokenizer here)
    --temperature  TEMPERATURE   default 0 = argmax
    --top-p        TOP_P         default 1
    --top-k        TOP_K         default unbounded
    --max-steps    MAX_STEPS     most tokens to generate, default: until the context is full

Verbs: ``generate`` (the default), ``inspect`` (print the typed configuration, as the reference
prints its meta before a run), ``random`` (write a model folder with random weights).
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys


def _env(name, cast, default):
    v = os.environ.get(name)
    if v is None:
        return default
    try:
        return cast(v)
    except ValueError:
        return default       # the reference ignores values it cannot parse (test-utils/src/lib.rs:60-65)


def parse_prompt(text: str):
    ids = [int(x) for x in re.split(r"[\s,]+", text.strip()) if x]
    if not ids:
        raise SystemExit("the prompt holds no token id")
    return ids


def _add_generate(ap):
    ap.add_argument("--model", default=os.environ.get("TEST_MODEL"))
    ap.add_argument("--devices", default=os.environ.get("DEVICES", "0"))
    ap.add_argument("--prompt", action="append", default=None,
                    help="token ids; give the option several times for a batch of prompts")
    ap.add_argument("--prompt-file", default=None, help="one prompt of token ids per line")
    ap.add_argument("--temperature", type=float, default=_env("TEMPERATURE", float, 0.0))
    ap.add_argument("--top-p", type=float, default=_env("TOP_P", float, 1.0))
    ap.add_argument("--top-k", type=int, default=_env("TOP_K", int, 0))
    ap.add_argument("--max-steps", type=int, default=_env("MAX_STEPS", int, None))
    ap.add_argument("--stop", default=None, help="stop token ids (default: the model's eos)")
    ap.add_argument("--seed", type=int, default=0, help="sampler seed")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-tokens", type=int, default=None, help="cache size in tokens")
    ap.add_argument("--max-batch", type=int, default=None)
    ap.add_argument("--json", action="store_true", help="print one JSON object instead of text")


def cmd_generate(args) -> int:
    if not args.model:
        print("TEST_MODEL not set", file=sys.stderr)     # test-utils/src/lib.rs:50-53
        return 2
    import transformer_b200 as tb
    prompts = []
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [parse_prompt(line) for line in f if line.strip()]
    for p in args.prompt or []:
        prompts.append(parse_prompt(p))
    if not prompts:
        env = os.environ.get("PROMPT")
        if env is None:
            raise SystemExit("no prompt: give --prompt (token ids) or set PROMPT")
        prompts.append(parse_prompt(env))
    sample_args = tb.SampleArgs(args.temperature, args.top_p, args.top_k)
    meta = tb.read_config(args.model)
    steps = args.max_steps
    need = sum((len(p) + (steps if steps is not None else 0) + 63) // 64 * 64 for p in prompts)
    max_tokens = args.max_tokens or max(need, 4096)
    engine = tb.load(args.model, dtype=args.dtype, device=f"cuda:{int(args.devices)}", max_tokens=max_tokens)
    stops = None if args.stop is None else parse_prompt(args.stop)
    res = tb.generate(engine, prompts, max_steps=steps, sample_args=sample_args, stop_tokens=stops,
                      seed=args.seed, max_batch=args.max_batch)
    if args.json:
        print(json.dumps({"tokens": res.tokens, "finished": res.finished,
                          "prefill_tokens": res.timing.prefill_tokens, "prefill_s": res.timing.prefill_seconds,
                          "decode_tokens": res.timing.decode_tokens, "decode_s": res.timing.decode_seconds}))
    else:
        print(sample_args)
        for p, t, w in zip(prompts, res.tokens, res.finished):
            print(" ".join(map(str, p)), "->", " ".join(map(str, t)), f"[{w}]")
        print()
        print(res.timing.table())
    return 0


def cmd_inspect(args) -> int:
    import transformer_b200 as tb
    from .config.registry import architecture_for
    cfg = tb.read_config(args.model)
    arch = architecture_for(cfg)
    meta = arch.config_cls.from_dict(cfg)
    print(f"architecture: {arch.name}")
    print(meta)
    return 0


def cmd_random(args) -> int:
    import transformer_b200 as tb
    with open(args.config) as f:
        cfg = json.load(f)
    tb.write_random_model(args.out, cfg, seed=args.seed, dtype=args.dtype, std=args.std)
    print(args.out)
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0].startswith("-"):
        argv = ["generate"] + argv
    ap = argparse.ArgumentParser(prog="transformer_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="verb", required=True)
    _add_generate(sub.add_parser("generate", help="generate tokens after the given prompts"))
    p = sub.add_parser("inspect", help="print the typed configuration of a model folder")
    p.add_argument("--model", default=os.environ.get("TEST_MODEL"), required=os.environ.get("TEST_MODEL") is None)
    p = sub.add_parser("random", help="write a model folder with random weights")
    p.add_argument("--config", required=True, help="a config.json")
    p.add_argument("--out", required=True)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--std", type=float, default=0.02)
    args = ap.parse_args(argv)
    return {"generate": cmd_generate, "inspect": cmd_inspect, "random": cmd_random}[args.verb](args)


if __name__ == "__main__":
    sys.exit(main())
