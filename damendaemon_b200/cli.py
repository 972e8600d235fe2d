"""Command line in the reference's manner (damendaemon/cli.py:81-91,111-119,326-333):

    python -m damendaemon_b200 run PATH --prompt TEXT --raw [--max-tokens N] [--context N]
                                   [--kv-cache-tokens N] [--no-graph] [--device cuda]
    python -m damendaemon_b200 init-random CONFIG.json OUT --seed S [--dtype bfloat16]

``run`` prints text deltas (token ids when the folder has no tokenizer) to standard output and
the final usage/timing JSON to standard error. GPT-2 has no chat template, so ``--raw`` is the
only prompt mode (docs/models.md:64-65 of the reference). Added here: --prompt-ids, --dtype,
--temperature, --top-p, --top-k, --seed, --ignore-eos, --page-size, --prefill-chunk-size.
"""
from __future__ import annotations

import argparse
import json
import sys


def build_parser():
    parser = argparse.ArgumentParser(prog="damendaemon_b200", description="B200-native single-GPU inference engine")
    commands = parser.add_subparsers(dest="command", required=True)
    run = commands.add_parser("run", help="generate from a local model directory")
    run.add_argument("path", help="local model directory (config.json + model.safetensors)")
    prompt = run.add_mutually_exclusive_group(required=True)
    prompt.add_argument("--prompt", help="prompt text (needs tokenizer.json in the model directory)")
    prompt.add_argument("--prompt-ids", help="prompt as comma-separated token ids")
    run.add_argument("--raw", action="store_true", help="use the prompt directly without a chat template (the only mode)")
    run.add_argument("--max-tokens", type=int, default=128)
    run.add_argument("--context", type=int, default=1024)
    run.add_argument("--kv-cache-tokens", type=int, help="shared KV token budget, a multiple of the page size")
    run.add_argument("--no-graph", action="store_true", help="do not replay decode steps from CUDA graphs")
    run.add_argument("--device", choices=("cuda",), default="cuda")
    run.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    run.add_argument("--temperature", type=float, default=0)
    run.add_argument("--top-p", type=float, default=1)
    run.add_argument("--top-k", type=int, default=0)
    run.add_argument("--seed", type=int)
    run.add_argument("--ignore-eos", action="store_true")
    run.add_argument("--page-size", type=int, default=16)
    run.add_argument("--prefill-chunk-size", type=int, default=0, help="prompt token budget per step; 0 disables")
    init = commands.add_parser("init-random", help="write a model folder with seeded random weights")
    init.add_argument("config", help="a config.json with the architecture's own keys")
    init.add_argument("out", help="folder to create")
    init.add_argument("--seed", type=int, default=0)
    init.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16", help="how matrices are stored")
    return parser


def main(argv=None):
    args = build_parser().parse_args(argv)
    if args.command == "init-random":
        from .config import read_config_file
        from .weights import write_random_model
        folder = write_random_model(args.out, read_config_file(args.config), args.seed, args.dtype)
        print(folder)
        return 0
    if args.prompt is not None and not args.raw:
        print("error: this architecture has no chat template; pass --raw", file=sys.stderr)
        return 2
    from .runtime import Runtime
    if args.kv_cache_tokens is not None and args.kv_cache_tokens % args.page_size:
        print("error: --kv-cache-tokens must be a multiple of the page size", file=sys.stderr)
        return 2
    runtime = Runtime(args.path, args.context, dtype=args.dtype, kv_cache_tokens=args.kv_cache_tokens, max_batch=1,
                      page_size=args.page_size, use_graph=not args.no_graph, prefill_chunk_size=args.prefill_chunk_size)
    prompt = args.prompt if args.prompt is not None else [int(x) for x in args.prompt_ids.split(",") if x.strip()]
    for event in runtime.generate(prompt, args.max_tokens, ignore_eos=args.ignore_eos, temperature=args.temperature,
                                  top_p=args.top_p, top_k=args.top_k, seed=args.seed):
        if "token" in event:
            print(event["text"] if runtime.tokenizer is not None else f"{event['token']} ", end="", flush=True)
        else:
            print()
            print(json.dumps(event), file=sys.stderr)
    return 0
