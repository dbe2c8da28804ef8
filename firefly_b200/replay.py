"""Trace replay: feed given token ids through a model step by step, write logits.

Nothing is sampled and nothing is scheduled here: the trace *is* the schedule.
Each input line is one step,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

and drives the engine's own model, step function, cache manager and kernels,
the ones generation uses.  For a step in which logits are wanted the file
``<out>/<step>.f32`` receives them as little-endian float32 [wanted, vocab], in
the order of the entries and of each entry's ``want``.  After every step the
line ``done <step>`` is printed and flushed.  The reference has no such tool
(its only way in is text over gRPC).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, Optional

import numpy as np
import torch

from .cache.manager import CacheManager, OutOfPages, RequestCache, plan_groups
from .engine.loading import load_model
from .engine.runner import ModelRunner, StepEntry, StepError

PAGE_ROUNDING = 64   # a request's token count is rounded up to this for --max-tokens


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page (divides 64)")
    ap.add_argument("--max-requests", type=int, default=16, help="most live requests")
    ap.add_argument("--device", default="cuda:0")
    return ap


class ReplaySession:
    """A model, its cache and its step function, driven one trace step at a time."""

    def __init__(self, model_dir: Optional[str] = None, *, dtype: str = "bfloat16", max_tokens: int,
                 block_size: int = 16, max_requests: int = 16, device: str = "cuda:0", model=None):
        """``model_dir``: a model folder; or ``model``: an already bound DecoderModel."""
        if block_size <= 0 or PAGE_ROUNDING % block_size:
            raise ValueError(f"block size must divide {PAGE_ROUNDING}")
        if model is None:
            self.model, self.config = load_model(model_dir, dtype=dtype, device=device)
        else:
            self.model, self.config = model, None
        self.max_tokens = max_tokens
        # every cache group holds max_tokens tokens in pages of its own size
        slot_specs = self.model.cache_slot_specs()
        counts = []
        for spec, _, bs in plan_groups(slot_specs, block_size):
            if PAGE_ROUNDING % bs:
                raise ValueError(f"a cache group's page size {bs} does not divide {PAGE_ROUNDING}")
            counts.append(-(-max_tokens // bs))
        self.cache = CacheManager(slot_specs, block_size=block_size, num_blocks=counts, max_requests=max_requests)
        self.cache.allocate_storage(self.model.rt.dtype, self.model.rt.device)
        max_len = min(self.model.spec.max_positions, -(-max_tokens // block_size) * block_size)
        if self.cache.groups and all(g.spec.window is not None for g in self.cache.groups):
            max_len = self.model.spec.max_positions     # windows give pages back: length is not bounded by the pool
        self.runner = ModelRunner(self.model, self.cache, max_model_len=max_len)
        self.live: Dict[str, RequestCache] = {}

    def run_step(self, rec) -> Optional[np.ndarray]:
        """One trace step.  Returns float32 [wanted, vocab], or None when nothing
        was wanted.  Raises OutOfPages when the pool cannot hold the step."""
        entries = []
        for ent in rec.get("entries", []):
            rid = str(ent["id"])
            tokens = [int(t) for t in ent["tokens"]]
            rc = self.live.get(rid)
            if rc is None:
                rc = self.cache.admit(rid)
                self.live[rid] = rc
            if not self.cache.grow(rc, rc.num_tokens + len(tokens)):
                raise OutOfPages(f"step {rec.get('step')}: out of cache pages for request '{rid}' "
                                 f"({rc.num_tokens}+{len(tokens)} tokens; pool of {self.max_tokens})")
            entries.append(StepEntry(rc, tokens, [int(w) for w in ent.get("want", [])]))
        logits = self.runner.step(entries)
        out = None
        if logits.shape[0]:
            out = logits.detach().to("cpu", torch.float32).numpy().astype("<f4", copy=False)
        else:
            torch.cuda.synchronize()
        self.runner.check_status()
        for rid in rec.get("end", []):
            rc = self.live.pop(str(rid), None)
            if rc is not None:
                self.cache.free(rc)
        return out


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    os.makedirs(args.out, exist_ok=True)
    try:
        session = ReplaySession(args.model, dtype=args.dtype, max_tokens=args.max_tokens,
                                block_size=args.block_size, max_requests=args.max_requests,
                                device=args.device)
    except ValueError as e:
        print(f"trace_run: {e}", file=sys.stderr)
        return 2
    while True:
        line = sys.stdin.readline()
        if not line:
            break
        line = line.strip()
        if not line:
            continue
        try:
            rec = json.loads(line)
            if not isinstance(rec, dict) or "step" not in rec:
                raise ValueError("a step is a JSON object with 'step', 'entries' and 'end'")
        except ValueError as e:
            print(f"trace_run: bad input line: {e}", file=sys.stderr)
            return 4
        try:
            arr = session.run_step(rec)
        except OutOfPages as e:
            print(f"trace_run: {e}", file=sys.stderr)
            return 3
        except (StepError, KeyError, TypeError, ValueError) as e:
            print(f"trace_run: step {rec.get('step')}: {type(e).__name__}: {e}", file=sys.stderr)
            return 4
        if arr is not None:
            with open(os.path.join(args.out, f"{rec['step']}.f32"), "wb") as fh:
                fh.write(arr.tobytes())
        print(f"done {rec['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
