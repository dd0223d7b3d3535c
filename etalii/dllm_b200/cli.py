"""The command line, in the manner of the reference's `dllm` (src/etalii_dllm/cli.py:284-297, 357-431, 754-802):
global options before the subcommand, `generate` with the reference's option names and meanings, generated ids on
standard output and `fingerprint: ... tokens: ... finish: ...` on standard error. Prompts are token ids (this
library takes and returns ids; text is the tokenizer's business).

    dllm-b200 --model DIR [--dtype bfloat16|float32] [--device cuda:0] generate --prompt-ids 1,2,3 --max-tokens 64
    dllm-b200 --model DIR info
    dllm-b200 random --config CONFIG.json --seed 0 --out DIR
"""
from __future__ import annotations

import argparse
import json
import sys

MAX_CHOICES = 64


def _ids(text: str) -> list[int]:
    return [int(part) for part in text.replace(",", " ").split()]


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="dllm-b200", description="Llama generation on one B200")
    parser.add_argument("--model", help="folder with config.json and model.safetensors")
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    parser.add_argument("--cache-tokens", type=int, default=None, help="tokens the cache holds (default 4 contexts)")
    commands = parser.add_subparsers(dest="command", required=True)

    generate = commands.add_parser("generate", help="continue a prompt")
    generate.add_argument("--prompt-ids", action="append", default=[], metavar="IDS",
                          help="the prompt as token ids, comma or space separated (repeatable: one batch)")
    generate.add_argument("--prompt-file", help="a file with one prompt of token ids per line")
    generate.add_argument("--n", type=int, default=1,
                          help="generate N choices; choice i samples with seed SEED+i (default 1)")
    generate.add_argument("--max-tokens", type=int, default=64)
    generate.add_argument("--temperature", type=float, default=0.0)
    generate.add_argument("--top-k", type=int, default=0)
    generate.add_argument("--top-p", type=float, default=1.0)
    generate.add_argument("--seed", type=int, default=0)
    generate.add_argument("--min-p", type=float, default=0.0, help="drop tokens below MIN_P times the top one")
    generate.add_argument("--min-tokens", type=int, default=0, help="no stop token before this many tokens")
    generate.add_argument("--ignore-eos", action="store_true", help="write past the model's end-of-sequence")
    generate.add_argument("--stop-token-id", type=int, action="append", default=[],
                          help="also end at this token id (repeatable)")

    commands.add_parser("info", help="the model's configuration and size")

    random = commands.add_parser("random", help="write a model folder with seeded random weights")
    random.add_argument("--config", required=True, help="a config.json to take the sizes from")
    random.add_argument("--seed", type=int, default=0)
    random.add_argument("--out", required=True)
    random.add_argument("--std", type=float, default=0.02)
    return parser


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    from . import architectures  # noqa: F401
    from .config.registry import ConfigError, config_from_dict, load_config
    from .sampling.options import SamplingOptions

    if args.command == "random":
        from .weights.random_init import write_random_model

        try:
            with open(args.config, encoding="utf-8") as handle:
                config = config_from_dict(json.load(handle))
            print(write_random_model(args.out, config, args.seed, std=args.std))
        except (ValueError, OSError) as error:  # an unreadable file, bad JSON, a configuration that is refused
            print(f"error: {error}", file=sys.stderr)
            return 2
        return 0
    if not args.model:
        print("error: --model is required", file=sys.stderr)
        return 2
    try:
        config = load_config(args.model)
    except (ConfigError, OSError) as error:
        print(f"error: {error}", file=sys.stderr)
        return 2
    if args.command == "info":
        print(json.dumps({"model": args.model, "device": args.device, "dtype": args.dtype, **config.to_hf()},
                         indent=1))
        return 0

    try:
        prompts = [_ids(text) for text in args.prompt_ids]
        if args.prompt_file:
            with open(args.prompt_file, encoding="utf-8") as handle:
                prompts += [_ids(line) for line in handle if line.strip()]
    except (ValueError, OSError) as error:
        print(f"error: a prompt is a list of token ids: {error}", file=sys.stderr)
        return 2
    if not prompts:
        print("error: give --prompt-ids or --prompt-file", file=sys.stderr)
        return 2
    if not 1 <= args.n <= MAX_CHOICES:
        print(f"error: --n must be between 1 and {MAX_CHOICES}", file=sys.stderr)
        return 2
    try:
        options = SamplingOptions(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, seed=args.seed,
                                  min_p=args.min_p)
    except ValueError as error:
        print(f"error: {error}", file=sys.stderr)
        return 2
    from .engine.engine import Engine

    try:
        engine = Engine.from_folder(args.model, dtype=args.dtype, device=args.device, max_tokens=args.cache_tokens)
    except (ValueError, OSError, RuntimeError) as error:  # weights that do not fit, no CUDA device, a failed build
        print(f"error: {error}", file=sys.stderr)
        return 2
    try:
        for index, prompt in enumerate(prompts):
            # the N choices of one prompt run as one batch; choice i draws from the stream of seed + i
            results = engine.generate([prompt] * args.n, args.max_tokens, options, ignore_eos=args.ignore_eos,
                                      stop_token_ids=args.stop_token_id, min_tokens=args.min_tokens)
            for choice, result in enumerate(results):
                if args.n > 1:
                    print(f"--- choice {choice} (seed {options.for_choice(choice).seed})", file=sys.stderr)
                print(" ".join(str(t) for t in result.tokens))
                print(f"fingerprint: {result.fingerprint}  tokens: {len(result.tokens)}  "
                      f"finish: {result.finish_reason}", file=sys.stderr)
    except (ValueError, RuntimeError) as error:  # a prompt that is refused, a cache that is too small, a kernel error
        print(f"error: {error}", file=sys.stderr)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
