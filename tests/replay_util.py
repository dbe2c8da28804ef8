"""Helpers of the replay tests: model folders, traces in the four cuttings, and
the comparison with the plain implementation."""
from __future__ import annotations

import json
import os
import random
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

import plain_qwen3 as P


def write_model_dir(path: str, cfg: dict, weights: Dict[str, torch.Tensor], dtype: torch.dtype) -> str:
    """config.json + model.safetensors written with the safetensors library (not
    with the engine's own writer, so that its reader is checked against another
    implementation of the format)."""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    save_file({k: v.to(dtype).contiguous() for k, v in weights.items()},
              os.path.join(path, "model.safetensors"))
    return path


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    """max |got - want| over a row, relative to the row's largest |want|."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.max(np.abs(got - want)) / (np.max(np.abs(want)) + 1e-30))


TOL = {"float32": 1e-4, "bfloat16": 4e-2}


class Collected:
    """Logits rows by (request, absolute position)."""

    def __init__(self):
        self.rows: Dict[Tuple[str, int], np.ndarray] = {}

    def add(self, rid: str, pos: int, row: np.ndarray):
        assert (rid, pos) not in self.rows, f"position {pos} of {rid} asked twice"
        self.rows[(rid, pos)] = np.array(row, copy=True)


def run_trace(session, steps: List[dict]) -> Collected:
    """Run steps through a ReplaySession, keeping every wanted row by position."""
    got = Collected()
    done: Dict[str, int] = {}
    for rec in steps:
        arr = session.run_step(rec)
        k = 0
        for ent in rec["entries"]:
            base = done.get(ent["id"], 0)
            for w in ent.get("want", []):
                got.add(ent["id"], base + w, arr[k])
                k += 1
            done[ent["id"]] = base + len(ent["tokens"])
        for rid in rec.get("end", []):
            done.pop(rid, None)
        assert arr is None or k == arr.shape[0]
    return got


def compare(got: Collected, plain_logits: Dict[str, np.ndarray], tol: float, what: str = ""):
    worst = (0.0, None)
    for (rid, pos), row in got.rows.items():
        base = rid.split("#")[0]
        e = rel_err(row, plain_logits[base][pos])
        if e > worst[0]:
            worst = (e, (rid, pos))
    assert worst[0] <= tol, f"{what}: relative error {worst[0]:.3e} > {tol:g} first/worst at {worst[1]}"
    return worst[0]


# ------------------------------------------------------------------ traces --
def trace_whole(reqs: Dict[str, List[int]]) -> List[dict]:
    """Each request alone and whole: one step, logits everywhere."""
    steps = []
    for i, (rid, toks) in enumerate(reqs.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def trace_tail_decode(reqs: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of it in one step, the last ``tail`` tokens one by one."""
    steps, s = [], 0
    for rid, toks in reqs.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                      "end": []})
        s += 1
        for p in range(head, len(toks)):
            steps.append({"step": s, "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
            s += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(reqs: Dict[str, List[int]], sizes: Sequence[int] = (17, 5, 2, 9, 2, 31, 3, 2, 64)) -> List[dict]:
    """Portions of changing size, down to two tokens."""
    steps, s = [], 0
    for rid, toks in reqs.items():
        p, k = 0, 0
        while p < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - p)
            k += 1
            last = p + n == len(toks)
            steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[p:p + n],
                                                 "want": list(range(n))}], "end": [rid] if last else []})
            p += n
            s += 1
    return steps


def trace_mixed(reqs: Dict[str, List[int]], *, seed: int = 0, max_live: int = 4, prompt_frac: float = 0.6,
                sizes: Sequence[int] = (13, 2, 7, 21, 3, 2, 16)) -> List[dict]:
    """Up to ``max_live`` requests at once: portions of some beside single tokens
    of others; a request is sometimes left out of a step; requests end at
    different times so that their pages go to the ones that start later."""
    rng = random.Random(seed)
    waiting = list(reqs.items())
    live: Dict[str, dict] = {}
    steps, s = [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = {"toks": toks, "p": 0, "prompt": min(len(toks), max(2, int(len(toks) * prompt_frac))), "k": rng.randrange(7)}
        entries, end = [], []
        for rid, st in list(live.items()):
            if len(live) > 1 and rng.random() < 0.2:
                continue   # left out of this step
            toks, p = st["toks"], st["p"]
            if p < st["prompt"]:
                n = min(sizes[st["k"] % len(sizes)], st["prompt"] - p)
                st["k"] += 1
            else:
                n = 1
            entries.append({"id": rid, "tokens": toks[p:p + n], "want": list(range(n))})
            st["p"] = p + n
            if st["p"] == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"step": s, "entries": entries, "end": end})
            s += 1
    return steps


def peak_tokens(steps: List[dict], rounding: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up."""
    held: Dict[str, int] = {}
    peak = 0
    for rec in steps:
        for ent in rec["entries"]:
            held[ent["id"]] = held.get(ent["id"], 0) + len(ent["tokens"])
        peak = max(peak, sum(-(-v // rounding) * rounding for v in held.values()))
        for rid in rec.get("end", []):
            held.pop(rid, None)
    return peak


def make_requests(vocab: int, lengths: Sequence[int], seed: int) -> Dict[str, List[int]]:
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


def plain_all(cfg: dict, weights: Dict[str, torch.Tensor], reqs: Dict[str, List[int]], **kw) -> Dict[str, np.ndarray]:
    return {rid: P.forward(cfg, weights, toks, **kw).numpy() for rid, toks in reqs.items()}
