"""Command line of firefly_b200.

In the manner of the reference's ``firefly_server [model_dir] [--max-prefill-chunk-size N]``
(src/server.cu:83-97): the model folder is the positional argument (default
``qwen3``) and ``--max-prefill-chunk-size`` has the same meaning (its default, 256, holds
while requests are decoding; while none is, a prompt is not cut).  The reference then serves chat completions over gRPC; this program
generates from token ids given on the command line or in a file and prints one
JSON line per request.  ``--max-tokens`` defaults to the reference's 512
(src/server.cu:189).

    firefly MODEL_DIR --prompt-ids 1,2,3 --max-tokens 16
    firefly MODEL_DIR --prompts-file prompts.jsonl --temperature 0.8 --seed 1
    firefly --random config.json --seed 0 --prompt-len 64 --num-prompts 4 --max-tokens 16
    firefly --write-random-model OUT_DIR --config config.json --seed 0

A fault of the input or of the machine (no CUDA device, a folder without weights, tensors that do
not fit the configuration) ends with one line on stderr and exit code 1, not with a traceback.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="firefly", description="Qwen3 dense inference on one B200")
    ap.add_argument("model_dir", nargs="?", default="qwen3",
                    help="folder with config.json and model.safetensors (default: qwen3)")
    ap.add_argument("--max-prefill-chunk-size", type=int, default=None,
                    help="most prompt tokens of one request in one step (default: 256 while requests are "
                         "decoding, whole prompts while none is)")
    ap.add_argument("--prompt-ids", action="append", default=[],
                    help="a prompt as comma-separated token ids; may be given several times")
    ap.add_argument("--prompts-file", help="file with one JSON list of token ids per line")
    ap.add_argument("--prompt-len", type=int, default=None,
                    help="make --num-prompts prompts of this many seeded random token ids")
    ap.add_argument("--num-prompts", type=int, default=1, help="how many prompts --prompt-len makes (default 1)")
    ap.add_argument("--random", metavar="CONFIG.json", default=None,
                    help="no model folder: a model of this configuration with seeded random weights (--seed)")
    ap.add_argument("--max-tokens", type=int, default=512, help="new tokens per request (default 512)")
    ap.add_argument("--temperature", type=float, default=0.0, help="0 = greedy (default)")
    ap.add_argument("--seed", type=int, default=0, help="seed of temperature sampling / random weights")
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--eos-token-id", type=int, action="append", default=None,
                    help="end-of-sequence id (default: config.json's eos_token_id)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--weight-dtype", default="keep", choices=["keep", "engine"],
                    help="tensors stored in 32-bit: keep them (default) or narrow them to --dtype on the device")
    ap.add_argument("--kv-block-size", type=int, default=16)
    ap.add_argument("--num-kv-blocks", type=int, default=None)
    ap.add_argument("--max-batch-size", type=int, default=64, help="most active requests (default 64)")
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--max-model-len", type=int, default=None)
    ap.add_argument("--no-cuda-graphs", action="store_true")
    ap.add_argument("--no-overlap-decode", action="store_true",
                    help="read every decode step's tokens before the next step is launched")
    ap.add_argument("--write-random-model", metavar="DIR",
                    help="write config.json and model.safetensors with seeded random weights, then exit")
    ap.add_argument("--config", help="config.json for --write-random-model")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.write_random_model:
        import torch
        from .models import config_from_dict
        from .weights import write_random_model
        if not args.config:
            print("firefly: --write-random-model needs --config CONFIG.json", file=sys.stderr)
            return 2
        with open(args.config) as fh:
            cfg = config_from_dict(json.load(fh))
        dt = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
        write_random_model(cfg, args.seed, args.write_random_model, dtype=dt)
        print(json.dumps({"written": args.write_random_model, "seed": args.seed, "dtype": args.dtype}))
        return 0

    prompts: List[List[int]] = []
    for p in args.prompt_ids:
        prompts.append([int(x) for x in p.replace(" ", "").split(",") if x])
    if args.prompts_file:
        with open(args.prompts_file) as fh:
            for line in fh:
                line = line.strip()
                if line:
                    prompts.append([int(x) for x in json.loads(line)])
    try:
        model = args.model_dir
        if args.random:
            from .models import config_from_dict
            with open(args.random) as fh:
                model = config_from_dict(json.load(fh))
        if args.prompt_len:
            import random
            if args.random:
                vocab = model.vocab_size
            else:
                from .models import load_config
                vocab = load_config(args.model_dir).vocab_size
            rng = random.Random(args.seed)
            prompts += [[rng.randrange(vocab) for _ in range(args.prompt_len)] for _ in range(args.num_prompts)]
        if not prompts:
            print("firefly: no prompt given (--prompt-ids, --prompts-file or --prompt-len)", file=sys.stderr)
            return 2
        from .entry import LLM
        llm = LLM(model, dtype=args.dtype, seed=args.seed, weight_dtype=args.weight_dtype,
                  max_prefill_chunk_size=args.max_prefill_chunk_size,
                  max_batch_size_limit=args.max_batch_size, max_num_batched_tokens=args.max_num_batched_tokens,
                  kv_block_size=args.kv_block_size, num_kv_blocks=args.num_kv_blocks,
                  max_model_len=args.max_model_len, eos_token_ids=args.eos_token_id,
                  use_cuda_graphs=not args.no_cuda_graphs, overlap_decode=not args.no_overlap_decode)
        outs = llm.generate(prompts, max_tokens=args.max_tokens, temperature=args.temperature, seed=args.seed,
                            ignore_eos=args.ignore_eos)
    except (RuntimeError, OSError, ValueError) as e:
        # ConfigError, WeightError, SafetensorsError and StepError are among these
        first = str(e).strip().splitlines()
        print(f"firefly: {first[0] if first else type(e).__name__}", file=sys.stderr)
        for line in first[1:]:
            print(f"  {line.strip()}", file=sys.stderr)
        return 1
    for i, (p, o) in enumerate(zip(prompts, outs)):
        print(json.dumps({"request": i, "prompt_tokens": len(p), "tokens": o}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
