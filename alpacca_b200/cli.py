"""Command line in the reference's manner (alpacca/cli.py:674-763).

    python -m alpacca_b200 run MODEL [PROMPT ...] [--ctx N] [--temp T] [--top-k K] [--top-p P]
                               [--repeat-penalty R] [--seed S] [--n-predict N]
    python -m alpacca_b200 show MODEL [--tensors]

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


# One table for the `run` command's options: the parser is built from it, and so are the sampler's
# options, so a flag and the field it sets cannot drift apart.  Names and short forms are the
# reference's (alpacca/cli.py:662-671); a sampler flag that is not given leaves the default of
# `SamplerParams` (alpacca/sample.py:12-19) in place.
#          flags                    type   sampler field      help
RUN_FLAGS = (
    (("--ctx", "-c"),               int,   None,              "context window (tokens)"),
    (("--temp",),                   float, "temperature",     "sampling temperature"),
    (("--top-k",),                  int,   "top_k",           None),
    (("--top-p",),                  float, "top_p",           None),
    (("--repeat-penalty",),         float, "repeat_penalty",  None),
    (("--seed", "-s"),              int,   "seed",            None),
    (("--n-predict", "-n"),         int,   None,              "max tokens to generate (-1 = until end)"),
)
RUN_DEFAULTS = {"ctx": 0, "n_predict": -1}      # flags that are no sampler option


def _dest(flags) -> str:
    return flags[0].lstrip("-").replace("-", "_")


def add_run_flags(parser: argparse.ArgumentParser) -> None:
    for flags, kind, field, text in RUN_FLAGS:
        parser.add_argument(*flags, type=kind, help=text,
                            default=None if field else RUN_DEFAULTS[_dest(flags)])
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                        help="bfloat16 (serving) or float32 (true 32-bit throughout)")


def sampler_params_from(args):
    from .sampling import SamplerParams
    given = {field: getattr(args, _dest(flags)) for flags, _, field, _ in RUN_FLAGS if field}
    return SamplerParams(**{k: v for k, v in given.items() if v is not None})


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
    results = generate(model, prompts, sampler_params_from(args), args.n_predict)
    for r in results:
        print(" ".join(str(t) for t in r.token_ids), flush=True)
        print(f"[{r.tokens} tokens, {r.tok_per_sec:.1f} tok/s]", file=sys.stderr)
    return 0


def cmd_show(args) -> int:
    """What a model folder holds, as the reference's `show` (alpacca/cli.py:240-259) does for an
    installed model: the configuration, the files and, with --tensors, the tensor table (the
    reference's --metadata).  It reads the folder only: no GPU is needed."""
    import json
    from pathlib import Path
    from .config import load_config
    from .engine.loading import build_model
    from .weights import FolderSource, check_names
    folder = Path(args.model)
    config = load_config(folder)
    print(json.dumps(config.to_dict(), indent=2))
    print(f"\nfiles in {folder}:")
    for f in sorted(folder.iterdir()):
        if f.is_file():
            print(f"  {f.name:<36} {f.stat().st_size / 2**20:10.1f} MiB")
    source = FolderSource(folder)
    try:
        table = source.table()
        model = build_model(config, device="cpu")
        check_names(model.param_specs(), table, where=str(folder))     # one error with everything that does not fit
        n = sum(int(__import__("math").prod(shape)) for _, shape in table.values())
        print(f"\n{config.architecture}: {len(model.spec.layers)} layers, {len(table)} tensors, "
              f"{n / 1e6:.1f}M parameters, positions up to {config.max_positions}; "
              f"every tensor the model expects is there with its shape")
        if args.tensors:
            print("\ntensors:")
            for name, (dtype, shape) in sorted(table.items()):
                print(f"  {name:<56} {dtype:<5} {list(shape)}")
    finally:
        source.close()
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
    add_run_flags(p)
    p.set_defaults(func=cmd_run)

    p = sub.add_parser("show", help="show a model folder's configuration, files and tensors")
    p.add_argument("model")
    p.add_argument("--tensors", action="store_true", help="list every tensor with dtype and shape")
    p.set_defaults(func=cmd_show)

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
    return _run_command(ap, args)


def _run_command(ap, args) -> int:
    """Exit codes as the reference's (alpacca/cli.py:751-763): 0, 1 with `alpacca_b200: error: ...`
    for what the user can mend, 130 when interrupted."""
    func = getattr(args, "func", None)
    if func is None:
        ap.print_help()
        return 0
    code, note = 0, None
    try:
        code = func(args)
    except (RuntimeError, ValueError) as fault:
        code, note = 1, f"alpacca_b200: error: {fault}"
    except KeyboardInterrupt:
        code, note = 130, ""
    if note is not None:
        print(note, file=sys.stderr)
    return code


if __name__ == "__main__":
    raise SystemExit(main())
