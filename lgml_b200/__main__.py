"""Command line: ``python -m lgml_b200 -m DIR --prompt-ids 1,2,3 -n 16``.

Flag names follow mischief/lgml's ``bin/lgml-server`` where it has them
(``:123-169``): ``-m/--model``, ``-c/--ctx`` (context size = cache pool),
``-np/--parallel`` (slots), ``-ub/--ubatch`` (prompt tokens per pass); the sampler
flags carry the sampler's option names (``src/sample.c:513-522``).  The engine is
tokens in, tokens out: prompts are comma-separated token ids, one ``--prompt-ids``
per request.
"""
from __future__ import annotations

import argparse
import json
import sys
import tempfile


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="lgml_b200", description="generate token ids with the B200 Llama engine")
    ap.add_argument("-m", "--model", help="model folder (config.json + model.safetensors)")
    ap.add_argument("--random-config", help="a config.json to run with random weights instead of a model folder")
    ap.add_argument("--write-random", metavar="DIR", help="with --random-config: write the random model folder to DIR and exit")
    ap.add_argument("--seed", type=int, default=None, help="sampler seed (request i uses seed + i); also the random-weights seed")
    ap.add_argument("-c", "--ctx", type=int, default=None, help="context size in tokens (default: the model's)")
    ap.add_argument("-np", "--parallel", type=int, default=4, help="slots: the most requests kept at once (default 4)")
    ap.add_argument("-ub", "--ubatch", type=int, default=512, help="prompt tokens per request per pass (default 512)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--prefix-cache", action="store_true", help="keep the full pages of ended requests findable: a prompt that begins like an earlier one computes only the rest")
    ap.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids; repeat for more requests")
    ap.add_argument("-n", "--max-tokens", type=int, default=16, help="new tokens per request")
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top-k", type=int, default=40)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--min-p", type=float, default=0.05)
    ap.add_argument("--repeat-penalty", type=float, default=1.0)
    ap.add_argument("--frequency-penalty", type=float, default=0.0)
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--repeat-last-n", type=int, default=64)
    ap.add_argument("--repeat-stop", type=int, default=256, help="equal tokens in a row that end a reply (0: off)")
    ap.add_argument("--stream", action="store_true", help="print every new token as 'request: id' as soon as it is known")
    ap.add_argument("--turn-csv", metavar="FILE", help="write one line per scheduler turn (seconds, tokens, decoded tokens, bytes copied) to FILE")
    ap.add_argument("--kernel-times", action="store_true", help="time every kernel class with CUDA events (steps run eagerly) and print microseconds per class to standard error")
    args = ap.parse_args(argv)

    from . import Engine, write_random_model
    from .config import config_from_dict

    cfg = None
    if args.random_config:
        cfg = config_from_dict(json.loads(open(args.random_config).read()))
        if args.write_random:
            write_random_model(args.write_random, cfg, args.seed or 0)
            print(args.write_random)
            return 0
    if not args.model and cfg is None:
        ap.error("give -m DIR or --random-config FILE")
    if not args.prompt_ids:
        ap.error("give at least one --prompt-ids")
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in args.prompt_ids]
    eng = Engine(args.model, config=cfg, random_weights=args.seed or 0, dtype=args.dtype, n_ctx=args.ctx, slots=args.parallel,
                 ubatch=args.ubatch, repeat_stop_tokens=args.repeat_stop, prefix_cache=args.prefix_cache)
    import contextlib

    from . import ops

    with (ops.KernelTimes() if args.kernel_times else contextlib.nullcontext()) as kt:
        outs = eng.generate(prompts, max_tokens=args.max_tokens, seed=args.seed, temperature=args.temperature, top_k=args.top_k,
                            top_p=args.top_p, min_p=args.min_p, repeat_penalty=args.repeat_penalty,
                            frequency_penalty=args.frequency_penalty, presence_penalty=args.presence_penalty,
                            repeat_last_n=args.repeat_last_n,
                            on_token=(lambda i, t: print(f"{i}: {t}", flush=True)) if args.stream else None)
    if kt is not None:
        tot = kt.totals()
        for name in sorted((k for k in tot if not k.endswith(" calls")), key=lambda k: -tot[k]):
            print(f"{name:28s} {tot[name]:12.1f} us in {tot[name + ' calls']} calls", file=sys.stderr)
    if args.turn_csv:
        eng.write_turn_csv(args.turn_csv)
    for o in outs:
        print(",".join(str(t) for t in o))
    return 0


if __name__ == "__main__":
    sys.exit(main())
