"""Closed-loop load on the engine's asynchronous interface: throughput, time to the
first token and time per output token.

The reference measures these through its gRPC server with
``benchmarks/benchmark_serving.py`` (``-c`` workers each keep one request
outstanding until ``-n`` requests are done; TTFT, TPOT = (total - TTFT) /
(tokens - 1), mean / median / P90 / P99, benchmarks/benchmark_serving.py:102-140).
This engine has no server, so the same load is put on ``Engine.async_generate``
and read back from its ``ResultQueue`` inside one process: option names, the
definitions of the figures and the printed report follow the reference's tool;
prompts are seeded random token ids of ``--prompt-len`` tokens where the
reference sends one fixed text.

    python -m firefly_b200.serving_bench MODEL_DIR -c 4 -n 20 --max-tokens 256
    python -m firefly_b200.serving_bench --config config.json --seed 0 -c 8 -n 64
"""
from __future__ import annotations

import argparse
import json
import random
import sys
import time
from typing import Dict, List, Optional

import numpy as np


def run_load(engine, result_queue, prompts: List[List[int]], *, concurrency: int, max_tokens: int,
             temperature: float = 0.0, ignore_eos: bool = True, timeout_s: float = 600.0) -> Dict[str, object]:
    """Keep ``concurrency`` requests outstanding until every prompt has been served.
    ``engine`` must have been built with ``result_queue``; it is started and stopped here."""
    from .sampling.params import SamplingParams
    if concurrency < 1:
        raise ValueError("concurrency must be >= 1")
    records: Dict[str, dict] = {}
    next_i = 0
    outstanding = 0

    def submit() -> None:
        nonlocal next_i, outstanding
        rid = f"bench-{next_i}"
        records[rid] = {"start": time.perf_counter(), "first": None, "end": None, "tokens": 0, "reason": None}
        engine.async_generate(rid, prompts[next_i], max_tokens,
                              SamplingParams(temperature=temperature, seed=next_i, max_tokens=max_tokens,
                                             ignore_eos=ignore_eos))
        next_i += 1
        outstanding += 1

    engine.start()
    t0 = time.perf_counter()
    try:
        while next_i < len(prompts) and outstanding < concurrency:
            submit()
        while outstanding:
            out = result_queue.pop(timeout=1.0)
            now = time.perf_counter()
            if out is None:
                if now - t0 > timeout_s:
                    raise TimeoutError(f"no result for {timeout_s} s with {outstanding} requests outstanding")
                continue
            rec = records[out.request_id]
            if out.new_tokens:
                if rec["first"] is None:
                    rec["first"] = now
                rec["tokens"] += len(out.new_tokens)
            if out.is_finished:
                rec["end"] = now
                rec["reason"] = out.finish_reason
                outstanding -= 1
                if next_i < len(prompts):
                    submit()
    finally:
        engine.stop()
    total = time.perf_counter() - t0
    ok = [r for r in records.values() if r["end"] is not None and not str(r["reason"] or "").startswith("error")]
    ttft = [r["first"] - r["start"] for r in ok if r["first"] is not None]
    tpot = [(r["end"] - r["first"]) / (r["tokens"] - 1) for r in ok if r["tokens"] > 1]
    tokens = sum(r["tokens"] for r in ok)

    def stats(xs: List[float]) -> Optional[Dict[str, float]]:
        if not xs:
            return None
        return {"mean": float(np.mean(xs)), "median": float(np.median(xs)),
                "p90": float(np.percentile(xs, 90)), "p99": float(np.percentile(xs, 99))}
    return {"num_requests": len(prompts), "successful": len(ok), "failed": len(prompts) - len(ok),
            "total_time_s": total, "total_tokens": tokens, "tokens_per_s": tokens / total,
            "requests_per_s": len(ok) / total, "ttft_s": stats(ttft), "tpot_s": stats(tpot),
            "engine": dict(engine.stats)}


def report(res: Dict[str, object]) -> str:
    """The reference tool's report (benchmarks/benchmark_serving.py:119-140)."""
    lines = ["--- Benchmark Results ---",
             f"Total Requests:      {res['num_requests']}",
             f"Successful Requests: {res['successful']}",
             f"Failed Requests:     {res['failed']}",
             f"Total Time:          {res['total_time_s']:.2f} s",
             f"Total Tokens:        {res['total_tokens']}",
             f"Throughput:          {res['tokens_per_s']:.2f} tokens/s",
             f"Request Throughput:  {res['requests_per_s']:.2f} req/s"]
    t = res["ttft_s"]
    if t:
        lines += ["", "--- Time To First Token (TTFT) ---",
                  f"Mean TTFT:           {t['mean']:.4f} s", f"Median TTFT:         {t['median']:.4f} s",
                  f"P90 TTFT:            {t['p90']:.4f} s", f"P99 TTFT:            {t['p99']:.4f} s"]
    t = res["tpot_s"]
    if t:
        lines += ["", "--- Time Per Output Token (TPOT) ---",
                  f"Mean TPOT:           {t['mean'] * 1000:.2f} ms/token",
                  f"Median TPOT:         {t['median'] * 1000:.2f} ms/token",
                  f"P90 TPOT:            {t['p90'] * 1000:.2f} ms/token",
                  f"P99 TPOT:            {t['p99'] * 1000:.2f} ms/token"]
    return "\n".join(lines)


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="firefly_b200.serving_bench",
                                 description="closed-loop load on the engine: throughput, TTFT, TPOT")
    ap.add_argument("model_dir", nargs="?", default=None, help="folder with config.json and model.safetensors")
    ap.add_argument("--config", help="config.json of a model with seeded random weights (instead of model_dir)")
    ap.add_argument("--seed", type=int, default=0, help="seed of the random weights and of the prompts")
    ap.add_argument("-c", "--concurrency", type=int, default=4, help="requests kept outstanding (default 4)")
    ap.add_argument("-n", "--num-requests", type=int, default=20, help="requests in total (default 20)")
    ap.add_argument("--max-tokens", type=int, default=256, help="new tokens per request (default 256)")
    ap.add_argument("--prompt-len", type=int, default=128, help="tokens per prompt (random ids)")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--stop-at-eos", action="store_true", help="end requests at config.json's eos_token_id")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-prefill-chunk-size", type=int, default=None,
                    help="most prompt tokens of one request in one step (default: the engine's own choice)")
    ap.add_argument("--max-batch-size", type=int, default=64)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--kv-block-size", type=int, default=16)
    ap.add_argument("--num-kv-blocks", type=int, default=None)
    ap.add_argument("--max-model-len", type=int, default=None)
    ap.add_argument("--json", action="store_true", help="print the figures as one JSON line too")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if (args.model_dir is None) == (args.config is None):
        print("serving_bench: give a model folder or --config CONFIG.json", file=sys.stderr)
        return 2
    from .engine.engine import Engine, EngineOptions, ResultQueue
    from .engine.loading import load_model, random_model
    raw = None
    if args.model_dir is not None:
        model, config = load_model(args.model_dir, dtype=args.dtype)
        import os
        with open(os.path.join(args.model_dir, "config.json")) as fh:
            raw = json.load(fh)
    else:
        from .models import config_from_dict
        with open(args.config) as fh:
            raw = json.load(fh)
        config = config_from_dict(raw)
        model = random_model(config, args.seed, dtype=args.dtype)
    need = args.prompt_len + args.max_tokens
    opts = EngineOptions(max_prefill_chunk_size=args.max_prefill_chunk_size,
                         max_batch_size_limit=args.max_batch_size,
                         max_num_batched_tokens=args.max_num_batched_tokens,
                         kv_block_size=args.kv_block_size, num_kv_blocks=args.num_kv_blocks,
                         max_model_len=args.max_model_len)
    queue = ResultQueue()
    engine = Engine(model, config, result_queue=queue, options=opts, raw_config=raw)
    if need > engine.max_model_len:
        print(f"serving_bench: prompt + new tokens ({need}) exceed the engine's length {engine.max_model_len}",
              file=sys.stderr)
        return 2
    rng = random.Random(args.seed)
    V = model.spec.vocab_size
    prompts = [[rng.randrange(V) for _ in range(args.prompt_len)] for _ in range(args.num_requests)]
    print(f"Starting benchmark with {args.concurrency} concurrent requests, {args.num_requests} total requests.")
    res = run_load(engine, queue, prompts, concurrency=args.concurrency, max_tokens=args.max_tokens,
                   temperature=args.temperature, ignore_eos=not args.stop_at_eos)
    print()
    print(report(res))
    if args.json:
        print(json.dumps(res))
    return 0 if res["failed"] == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
