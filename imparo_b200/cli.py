"""Command line, in the manner of the reference's token-id instrument and server flags:

    python -m imparo_b200 -m MODEL_DIR [--decode N] [--repeat N] [-c CTX] [-np PARALLEL]
                          [--temperature T] [--seed S] [--dtype bfloat16|float32]
                          (TOKEN... | -t FILE | --prompt-len N [--batch B])

Names and meanings follow the reference where it has them: `-m/--model`, `-c/--ctx`
(context length, default 4096), `-np/--parallel` (requests that decode at once)
(imparo-server/src/main.rs:178-240); `--decode N` (N new tokens after the prompt, the
token trail is printed), `--repeat N`, token ids as arguments or `-t FILE`
(imparo-model/src/bin/imparo-forward.rs:1036-1075,1343-1358).  The request fields
max_tokens and temperature map to --decode and --temperature.  `--random CONFIG.json`
draws random weights for a configuration instead of reading a model folder.
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="python -m imparo_b200", description="LFM2 generation from token ids on one B200.")
    ap.add_argument("-m", "--model", help="folder with config.json and model.safetensors")
    ap.add_argument("--random", metavar="CONFIG.json", help="random weights for this config.json instead of a model folder")
    ap.add_argument("--write-random", metavar="DIR", help="with --random: write the model folder DIR and exit")
    ap.add_argument("--seed", type=int, default=0, help="seed of random weights and of temperature sampling")
    ap.add_argument("--dtype", default=None, choices=["bfloat16", "float32", "bf16", "fp32"], help="default bfloat16")
    ap.add_argument("-c", "--ctx", type=int, default=None, help="context length: most positions one request may reach (default 4096)")
    ap.add_argument("--config-file", metavar="FILE.json", help="engine settings (ctx, parallel, page_size, switches, ...); a flag "
                    "wins over an IMPARO_* variable, which wins over this file")
    ap.add_argument("-np", "--parallel", type=int, default=None, help="requests that decode at once")
    ap.add_argument("--decode", type=int, default=16, metavar="N", help="new tokens per request (the request's max_tokens)")
    ap.add_argument("--repeat", type=int, default=1, metavar="N", help="run the same requests N times (determinism check)")
    ap.add_argument("--temperature", type=float, default=0.0, help="0 is greedy")
    ap.add_argument("-t", "--tokens-file", metavar="FILE", help="token ids, whitespace-separated, one prompt per line")
    ap.add_argument("--prompt-len", type=int, help="uniform-random prompts of this length instead of given ids")
    ap.add_argument("--batch", type=int, default=1, help="with --prompt-len: how many prompts")
    ap.add_argument("--page-size", type=int, default=None, help="positions per cache page (default 16)")
    ap.add_argument("--num-pages", type=int, default=None)
    ap.add_argument("--max-step-tokens", type=int, default=None, help="token budget of one step (default 2048)")
    ap.add_argument("--probe-layer", type=int, default=None, metavar="I",
                    help="print rms, sum and first values of the stages of schedule entry I (for comparing engines; slow)")
    ap.add_argument("--json", action="store_true", help="print one JSON line with tokens and timings")
    ap.add_argument("tokens", nargs="*", type=int, help="prompt token ids")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if bool(args.model) == bool(args.random):
        print("give exactly one of -m/--model and --random", file=sys.stderr)
        return 2
    config = None
    if args.random:
        with open(args.random) as f:
            config = json.load(f)
        if args.write_random:
            from .weights import write_random_model
            write_random_model(args.write_random, config, args.seed, "float32" if args.dtype in ("float32", "fp32") else "bfloat16")
            print(f"wrote {args.write_random}")
            return 0
    prompts = []
    if args.tokens_file:
        with open(args.tokens_file) as f:
            prompts = [[int(x) for x in line.split()] for line in f if line.strip()]
    elif args.tokens:
        prompts = [list(args.tokens)]
    from .engine import Engine
    parallel = args.parallel or max(1, len(prompts) if prompts else args.batch)
    t0 = time.perf_counter()
    engine = Engine(args.model, config=config, seed=args.seed, dtype=args.dtype, ctx=args.ctx, parallel=parallel,
                    page_size=args.page_size, num_pages=args.num_pages, max_step_tokens=args.max_step_tokens, probe_layer=args.probe_layer,
                    config_file=args.config_file)
    load_s = time.perf_counter() - t0
    if not prompts:
        if not args.prompt_len:
            print("give at least one token id (arguments, -t FILE, or --prompt-len N)", file=sys.stderr)
            return 2
        import numpy as np
        rng = np.random.default_rng(args.seed)
        prompts = [rng.integers(0, engine.vocab_size, args.prompt_len).tolist() for _ in range(args.batch)]
    outs = []
    for rep in range(args.repeat):
        t1 = time.perf_counter()
        outs.append(engine.generate(prompts, max_tokens=args.decode, temperature=args.temperature,
                                    seed=[args.seed + i for i in range(len(prompts))]))
        dt = time.perf_counter() - t1
        n_new = sum(len(o) for o in outs[-1])
        if not args.json:
            for i, o in enumerate(outs[-1]):
                print(f"rep {rep} request {i}: prompt {len(prompts[i])} tokens -> " + " ".join(map(str, o)))
            print(f"rep {rep}: {n_new} tokens in {dt * 1e3:.1f} ms ({n_new / dt:.1f} tok/s), load {load_s:.1f} s",
                  file=sys.stderr)
    same = all(o == outs[0] for o in outs)
    if args.repeat > 1 and not args.json:
        print(f"determinism: {'1' if same else 'several'} distinct outputs over {args.repeat} reps")
    if args.json:
        print(json.dumps({"tokens": outs[0], "repeat_equal": same, "load_s": round(load_s, 3), "stats": engine.stats()},
                         default=str))
    return 0 if same else 1
