"""Command line in the reference's manner (alpacca/cli.py:674-763).

    python -m alpacca_b200 run MODEL [PROMPT ...] [--ctx N] [--temp T] [--top-k K] [--top-p P]
                               [--repeat-penalty R] [--seed S] [--n-predict N]

The flags are the reference's (`_add_model_flags`, alpacca/cli.py:662-671)
with its defaults (alpacca/sample.py:12-19).  MODEL is a model folder; a
prompt is token ids (there is no tokenizer here): numbers separated by spaces
or commas; `/` separates several prompts, which then run as one batch.  The
generated ids go to standard output, one line per prompt, and
`[N tokens, X tok/s]` to standard error as in alpacca/cli.py:278.  Errors:
`alpacca_b200: error: ...` and exit code 1 (:759-763).
"""
from __future__ import annotations

import argparse
import sys

from . import __version__


def _add_model_flags(p: argparse.ArgumentParser) -> None:
    p.add_argument("--ctx", "-c", type=int, default=0, help="context window (tokens)")
    p.add_argument("--temp", type=float, default=None, help="sampling temperature")
    p.add_argument("--top-k", type=int, default=None)
    p.add_argument("--top-p", type=float, default=None)
    p.add_argument("--repeat-penalty", type=float, default=None)
    p.add_argument("--seed", "-s", type=int, default=None)
    p.add_argument("--n-predict", "-n", type=int, default=-1, help="max tokens to generate (-1 = until end)")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                   help="bfloat16 (serving) or float32 (true 32-bit throughout)")


def _sampler_params(args):
    from .sampling import SamplerParams
    p = SamplerParams()
    if args.temp is not None:
        p.temperature = args.temp
    if args.top_k is not None:
        p.top_k = args.top_k
    if args.top_p is not None:
        p.top_p = args.top_p
    if args.repeat_penalty is not None:
        p.repeat_penalty = args.repeat_penalty
    if args.seed is not None:
        p.seed = args.seed
    return p


def parse_prompts(words) -> list[list[int]]:
    text = " ".join(words).replace(",", " ")
    prompts = []
    for part in text.split("/"):
        try:
            prompts.append([int(w) for w in part.split()])
        except ValueError:
            raise ValueError("a prompt is a list of token ids (numbers separated by spaces or commas; "
                             "'/' between prompts); this library has no tokenizer") from None
    return prompts


def cmd_run(args) -> int:
    from .api import Model, generate
    prompts = parse_prompts(args.prompt)
    print(f"loading {args.model}...", file=sys.stderr)
    model = Model.load(args.model, n_ctx=args.ctx, dtype=args.dtype, max_batch=max(len(prompts), 1))
    print(model.describe(), file=sys.stderr)
    results = generate(model, prompts, _sampler_params(args), args.n_predict)
    for r in results:
        print(" ".join(str(t) for t in r.token_ids), flush=True)
        print(f"[{r.tokens} tokens, {r.tok_per_sec:.1f} tok/s]", file=sys.stderr)
    return 0


def cmd_make_random(args) -> int:
    import json
    from .engine.loading import write_random_model_dir
    cfg = json.loads(open(args.config).read())
    out = write_random_model_dir(args.out, cfg, args.seed, dtype=args.dtype)
    print(f"wrote {out}", file=sys.stderr)
    return 0


def cmd_replay(args) -> int:
    from .engine.trace import replay
    return replay(args.model, args.dtype, args.out, args.max_tokens, sys.stdin, sys.stdout)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="alpacca_b200",
                                 description="alpacca_b200 - Llama-style generation on one B200")
    ap.add_argument("--version", "-v", action="version", version=f"alpacca_b200 {__version__}")
    sub = ap.add_subparsers(dest="command", metavar="<command>")

    p = sub.add_parser("run", help="generate from a model folder (token ids in, token ids out)")
    p.add_argument("model")
    p.add_argument("prompt", nargs="*")
    _add_model_flags(p)
    p.set_defaults(func=cmd_run)

    p = sub.add_parser("make-random", help="write a model folder with random weights from a config.json")
    p.add_argument("config", help="a config.json of a registered architecture")
    p.add_argument("out", help="folder to write config.json and model.safetensors into")
    p.add_argument("--seed", "-s", type=int, default=0)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.set_defaults(func=cmd_make_random)

    p = sub.add_parser("replay", help="feed given token ids step by step and write logits (see bin/trace_run)")
    p.add_argument("--model", required=True)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True)
    p.add_argument("--max-tokens", type=int, required=True)
    p.set_defaults(func=cmd_replay)

    args = ap.parse_args(argv)
    if not args.command:
        ap.print_help()
        return 0
    try:
        return args.func(args)
    except KeyboardInterrupt:
        print("", file=sys.stderr)
        return 130
    except (RuntimeError, ValueError) as e:
        print(f"alpacca_b200: error: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    raise SystemExit(main())
