"""The command line, in the manner of the reference's `dllm` (src/etalii_dllm/cli.py:284-297, 357-431, 754-802):
global options before the subcommand, `generate` with the reference's option names and meanings, generated ids on
standard output and `fingerprint: ... tokens: ... finish: ...` on standard error. Prompts are token ids (this
library takes and returns ids; text is the tokenizer's business).

    dllm-b200 --model DIR [--dtype bfloat16|float32] [--device cuda:0] generate --prompt-ids 1,2,3 --max-tokens 64
    dllm-b200 --model DIR info
    dllm-b200 --model DIR [--dtype ...] replay --out DIR --max-tokens N < steps.jsonl
    dllm-b200 --model DIR [--dtype ...] bench [--batch 8] [--prompt-tokens 512] [--new-tokens 64] [--repeats 5]
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
                          help="the prompt as token ids, comma or space separated (repeatable: the prompts run "
                               "together as one batch, as far as the cache holds them)")
    generate.add_argument("--prompt-file", help="a file with one prompt of token ids per line (same batch)")
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

    replay = commands.add_parser("replay", help="feed token ids from standard input step by step and write logits "
                                                "(what bin/trace_run does)")
    replay.add_argument("--out", required=True, help="folder for <step>.f32 files")
    replay.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time, each rounded up to a multiple of 64")

    bench = commands.add_parser("bench", help="time whole generation calls on seeded random prompts: one warm-up, "
                                              "mean and sd of the repetitions, one JSON line")
    bench.add_argument("--batch", type=int, default=8)
    bench.add_argument("--prompt-tokens", type=int, default=512)
    bench.add_argument("--new-tokens", type=int, default=64)
    bench.add_argument("--repeats", type=int, default=5)
    bench.add_argument("--temperature", type=float, default=0.0)
    bench.add_argument("--seed", type=int, default=0)

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

    if args.command == "replay":
        from .replay import run

        try:
            return run(args.model, args.dtype, args.out, args.max_tokens, args.device)
        except (ValueError, OSError, RuntimeError, KeyError) as error:
            print(f"error: {error}", file=sys.stderr)
            return 2
    if args.command == "bench":
        return _bench(args, config)

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
        # every prompt's N choices, all prompts together, in ONE call: the engine cuts the list into as many batches
        # as the cache needs; choice c of every prompt draws from the stream of seed + c
        requests = [prompt for prompt in prompts for _ in range(args.n)]
        seeds = [options.for_choice(choice).seed for _ in prompts for choice in range(args.n)]
        results = engine.generate(requests, args.max_tokens, options, ignore_eos=args.ignore_eos,
                                  stop_token_ids=args.stop_token_id, min_tokens=args.min_tokens, seeds=seeds)
    except (ValueError, RuntimeError) as error:  # a prompt that is refused, a cache that is too small, a kernel error
        print(f"error: {error}", file=sys.stderr)
        return 2
    for index, result in enumerate(results):
        choice = index % args.n
        if len(prompts) > 1 and choice == 0:
            print(f"--- prompt {index // args.n}", file=sys.stderr)
        if args.n > 1:
            print(f"--- choice {choice} (seed {options.for_choice(choice).seed})", file=sys.stderr)
        print(" ".join(str(t) for t in result.tokens))
        print(f"fingerprint: {result.fingerprint}  tokens: {len(result.tokens)}  "
              f"finish: {result.finish_reason}", file=sys.stderr)
    return 0


def _bench(args, config) -> int:
    """`bench`: seeded random prompts of one length through `Engine.generate`, timed as a whole."""
    from .measure import measure_generation, random_prompts
    from .sampling.options import SamplingOptions

    if args.batch < 1 or args.prompt_tokens < 1 or args.new_tokens < 1 or args.repeats < 1:
        print("error: --batch, --prompt-tokens, --new-tokens and --repeats must be positive", file=sys.stderr)
        return 2
    from .engine.engine import Engine

    try:
        options = SamplingOptions(temperature=args.temperature, seed=args.seed)
        per_sequence = -(-(args.prompt_tokens + args.new_tokens) // 64) * 64
        engine = Engine.from_folder(args.model, dtype=args.dtype, device=args.device,
                                    max_tokens=args.cache_tokens or args.batch * per_sequence,
                                    max_length=per_sequence)
        prompts = random_prompts(engine.vocab_size, [args.prompt_tokens] * args.batch, args.seed)
        measured = measure_generation(engine, prompts, args.new_tokens, options, repeats=args.repeats)
    except (ValueError, OSError, RuntimeError) as error:
        print(f"error: {error}", file=sys.stderr)
        return 2
    print(json.dumps({"model": args.model, "dtype": args.dtype, "batch": args.batch,
                      "prompt_tokens": args.prompt_tokens, "new_tokens": args.new_tokens,
                      **{key: round(value, 6) if isinstance(value, float) else value
                         for key, value in measured.items()}}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
