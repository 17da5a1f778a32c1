"""Command line, in the manner of the reference's token-fed tools
(`gen_from_tokens -m MODEL --tokens FILE -n N [--ctx N]`, tools/baseline/gen_from_tokens.cpp:
11,39-44) with the sampling options of `boom_llm_sampling` under the names its binding gives
them (bindings/guile/scheme/sonicboom/inference.scm:586-620).

    python -m sonicboom_b200 generate -m DIR --tokens FILE -n 32 [--temperature 0.8 --seed 1 ...]
    python -m sonicboom_b200 random-model --config config.json --seed 7 --out DIR
    python -m sonicboom_b200 --version

`--tokens FILE` holds token ids separated by white space, one prompt a line; the generated
ids are printed one line per prompt, space separated.
"""
from __future__ import annotations

import argparse
import json
import sys


def _add_sampling(ap):
    ap.add_argument("-n", "--max-tokens", type=int, default=16, help="tokens to produce per prompt")
    ap.add_argument("--temperature", type=float, default=0.0, help="0 is greedy")
    ap.add_argument("--top-k", type=int, default=0, help="0 disables top-k truncation")
    ap.add_argument("--top-p", type=float, default=1.0, help="1 disables nucleus truncation")
    ap.add_argument("--min-p", type=float, default=0.0, help="0 disables min-p truncation")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--repeat-penalty", type=float, default=1.0)
    ap.add_argument("--repeat-last-n", type=int, default=64)
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--frequency-penalty", type=float, default=0.0)


def read_prompts(path: str) -> list:
    prompts = []
    with open(path) as fh:
        for line in fh:
            ids = [int(t) for t in line.split()]
            if ids:
                prompts.append(ids)
    if not prompts:
        raise SystemExit(f"tokens file empty: {path}")
    return prompts


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="sonicboom_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--version", action="store_true", help="print the build information and exit")
    sub = ap.add_subparsers(dest="command")
    g = sub.add_parser("generate", help="continue token-id prompts")
    g.add_argument("-m", "--model", required=True, help="folder with config.json and model.safetensors")
    g.add_argument("--tokens", required=True, help="file of token ids, one prompt a line")
    g.add_argument("--ctx", type=int, default=0,
                   help="cache size in tokens (default: what the prompts and -n need)")
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--device", default="cuda:0")
    g.add_argument("--ignore-eos", action="store_true", help="do not stop at the model's eos ids")
    g.add_argument("--stop", type=int, action="append", default=None, help="stop token id (repeatable)")
    _add_sampling(g)
    r = sub.add_parser("random-model", help="write a model folder with seeded random weights")
    r.add_argument("--config", required=True, help="config.json to build from")
    r.add_argument("--seed", type=int, required=True)
    r.add_argument("--out", required=True)
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--bias-std", type=float, default=None)
    r.add_argument("--norm-std", type=float, default=0.0)
    args = ap.parse_args(argv)
    if args.version:
        from .buildinfo import build_info_line
        print(build_info_line())
        return 0
    if args.command is None:
        ap.error("a command is required: generate or random-model")

    if args.command == "random-model":
        from .weights import write_random_model
        with open(args.config) as fh:
            cfg = json.load(fh)
        out = write_random_model(args.out, cfg, args.seed, args.std, args.bias_std, args.norm_std)
        print(out)
        return 0

    from . import llm
    from .sampling import Sampling
    prompts = read_prompts(args.tokens)
    model = llm.model_load(args.model, dtype=args.dtype, device=args.device)
    sampling = Sampling(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                        seed=args.seed, max_tokens=args.max_tokens, min_p=args.min_p,
                        repeat_penalty=args.repeat_penalty, repeat_last_n=args.repeat_last_n,
                        presence_penalty=args.presence_penalty,
                        frequency_penalty=args.frequency_penalty)
    outs = llm.generate_batch(model, prompts, sampling=sampling, stop_tokens=args.stop,
                              ignore_eos=args.ignore_eos, max_cache_tokens=args.ctx or None)
    for ids in outs:
        print(" ".join(str(t) for t in ids))
    return 0


if __name__ == "__main__":
    sys.exit(main())
