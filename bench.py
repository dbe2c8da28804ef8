#!/usr/bin/env python3
"""Benchmark of firefly_b200 on one B200: decode tokens per second of a
Qwen3-8B-shaped model (random weights, synthetic token ids), plus prefill
throughput, the decode step's memory roofline and batch-1 / batch-64 points.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers N] [--impl ours|reference]

One JSON line is printed.  ``value`` is device-timed (CUDA events around K
decode steps that run back to back from CUDA graphs, the sampled tokens fed to
the next step on the device); ``e2e`` is K steps through the Python entry
point's engine loop (``Engine.step``: scheduler, the step's metadata host ->
device from pinned memory, sampled tokens device -> host, every step), half of
them before and half after the device-timed bracket, because the step time
drifts upward over the first hundreds of steps at full power.  The decode step streams ~15 GB of weights, far
more than the 126 MB L2, so no extra flush is needed between timed iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


SHAPES = {   # BASELINE.json configs[2] (the metric), configs[3] and configs[4]
    "8b": dict(hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
               num_key_value_heads=8, tie_word_embeddings=False),
    "0.6b": dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
                 num_key_value_heads=8, tie_word_embeddings=True),
    "32b": dict(hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64,
                num_key_value_heads=8, tie_word_embeddings=False),
}


def load_shape(name: str = "8b"):
    """Layer sizes of a BASELINE.json shape (default configs[2], Qwen3-8B-shaped), as config.json keys."""
    base = dict(architectures=["Qwen3ForCausalLM"], head_dim=128, vocab_size=151936,
                max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1e6)
    base.update(SHAPES[name])
    return base


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as fh:
                raw = json.load(fh)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(raw.get(k), (int, float)):
                    out[k] = float(raw[k])
            out["source"] = "measured"
            return out
        except Exception:  # noqa: BLE001
            pass
    out = dict(FALLBACK_PEAKS)
    out["source"] = "fallback"
    return out


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", "0", "-lms", "200"], stdout=self.fh, stderr=subprocess.DEVNULL)
        except Exception:  # noqa: BLE001
            self.proc = None

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        self.fh.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as fh:
            for line in fh:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return None
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


REF_BIN = os.path.join(ROOT, "baseline", "_ref", "ref_bench")


def write_reference_model(folder: str, shape: dict, seed: int = 0) -> float:
    """A model folder the reference can load: config.json, model.safetensors (FP16, the only type its
    kernels run; matrices N(0, 0.02), norm weights 1 + N(0, 0.01), drawn tensor by tensor and written
    as they come, so the host never holds the model) and a tokenizer.json that gives every id a text
    (the reference's engine reports a token only when it has text for it).  Returns gigabytes written."""
    import struct

    import torch
    H, I, L, V = shape["hidden_size"], shape["intermediate_size"], shape["num_hidden_layers"], shape["vocab_size"]
    nq, nkv, d = shape["num_attention_heads"], shape["num_key_value_heads"], shape["head_dim"]
    tensors = [("model.embed_tokens.weight", (V, H)), ("model.norm.weight", (H,)), ("lm_head.weight", (V, H))]
    for i in range(L):
        p = f"model.layers.{i}"
        tensors += [(f"{p}.input_layernorm.weight", (H,)), (f"{p}.post_attention_layernorm.weight", (H,)),
                    (f"{p}.self_attn.q_proj.weight", (nq * d, H)), (f"{p}.self_attn.k_proj.weight", (nkv * d, H)),
                    (f"{p}.self_attn.v_proj.weight", (nkv * d, H)), (f"{p}.self_attn.o_proj.weight", (H, nq * d)),
                    (f"{p}.self_attn.q_norm.weight", (d,)), (f"{p}.self_attn.k_norm.weight", (d,)),
                    (f"{p}.mlp.gate_proj.weight", (I, H)), (f"{p}.mlp.up_proj.weight", (I, H)),
                    (f"{p}.mlp.down_proj.weight", (H, I))]
    header, off = {}, 0
    for name, shp in tensors:
        n = 2
        for x in shp:
            n *= x
        header[name] = {"dtype": "F16", "shape": list(shp), "data_offsets": [off, off + n]}
        off += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    with open(os.path.join(folder, "model.safetensors"), "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name, shp in tensors:
            x = torch.randn(shp, generator=gen, device="cuda", dtype=torch.float32)
            x = (1.0 + 0.01 * x) if len(shp) == 1 else 0.02 * x
            fh.write(x.to(torch.float16).cpu().numpy().tobytes())
    cfg = {k: shape[k] for k in ("architectures", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads", "head_dim", "vocab_size",
                                 "max_position_embeddings", "rms_norm_eps", "rope_theta")}
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    with open(os.path.join(folder, "tokenizer.json"), "w") as fh:
        json.dump({"model": {"vocab": {f"a{i}": i for i in range(V)}, "merges": []}}, fh)
    return off / 1e9


def _baseline_record() -> dict:
    """BASELINE.json beside this file (it names where the reference's sources lie), or nothing."""
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as fh:
            return json.load(fh)
    except (OSError, ValueError):
        return {}


def reference_arm(args) -> int:
    """The reference's own engine (built unmodified by baseline/build_reference.py into
    baseline/_ref/ref_bench) on the same shape and batch, fed through Engine::async_generate and timed
    from outside by the arrival of its tokens."""
    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    if args.gpus != 1:
        return unavailable("the reference runs on one GPU only (it has no multi-GPU path)")
    if not os.path.isfile(REF_BIN):
        src = os.environ.get("FIREFLY_REFERENCE") or _baseline_record().get("reference_path", "")
        if not src or not os.path.isdir(os.path.join(src, "src", "kernels")):
            return unavailable("baseline/_ref/ref_bench is not built and the reference's sources are not on this "
                               "machine (python baseline/build_reference.py builds it where they are)")
        try:
            subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "build_reference.py"), src], check=True,
                           stdout=subprocess.DEVNULL, stderr=subprocess.PIPE, text=True, timeout=1500)
        except Exception as e:  # noqa: BLE001
            tail = (getattr(e, "stderr", "") or str(e)).strip().splitlines()[-1:] or [str(e)]
            return unavailable(f"the reference's sources do not build here: {tail[0][:200]}")
    if args.dtype != "bfloat16":
        return unavailable("the reference has one element type (FP16 with FP16 accumulation)")
    if args.prompt_len % 16:
        return unavailable("the reference's prefill kernel reads past prompts that are no multiple of 16 tokens "
                           "(src/kernels/attention.cu:78,240); not run")
    import shutil

    import torch
    if not torch.cuda.is_available():
        return unavailable("no CUDA device on this machine")
    shape = load_shape(args.shape)
    full_layers = shape["num_hidden_layers"]
    if args.layers:
        shape["num_hidden_layers"] = args.layers
    K_steps, W = args.steps, max(args.warmup, 3)
    pk = peaks()
    folder = tempfile.mkdtemp(prefix="firefly_ref_model_")
    clocks = ClockSampler()
    try:
        t0 = time.time()
        gb = write_reference_model(folder, shape)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        write_s = time.time() - t0
        if not os.environ.get("FF_NO_CLOCKS"):
            clocks.start()
        proc = subprocess.run([REF_BIN, folder, "--batch", str(args.batch), "--prompt-len", str(args.prompt_len),
                               "--steps", str(K_steps), "--warmup", str(W)], capture_output=True, text=True,
                              timeout=1500)
        clock_info = clocks.stop()
        line = next((x for x in proc.stdout.splitlines() if x.startswith("REF_RESULT ")), None)
        if proc.returncode != 0 or line is None:
            tail = (proc.stderr.strip().splitlines() or proc.stdout.strip().splitlines() or ["no output"])[-1]
            return unavailable(f"the reference's engine ended with code {proc.returncode} on this machine: {tail[:300]}")
        r = json.loads(line[len("REF_RESULT "):])
    except subprocess.TimeoutExpired:
        clocks.stop()
        return unavailable("the reference's engine did not finish within 25 minutes")
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    L, H, I, V = shape["num_hidden_layers"], shape["hidden_size"], shape["intermediate_size"], shape["vocab_size"]
    nq, nkv, d = shape["num_attention_heads"], shape["num_key_value_heads"], shape["head_dim"]
    out = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-{args.shape.upper()}-shaped float16, {args.prompt_len}-token prompts)",
        "value": r["tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": K_steps, "warmup": W,
        "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16", "data": "synthetic", "impl": "reference",
        "config": {"model": f"Qwen3-{args.shape.upper()}-shaped random weights", "global_batch": args.batch,
                   "seq_len": args.context, "parallelism": "single GPU", "layers": L, "layers_of_config": full_layers,
                   "hidden": H, "q_heads": nq, "kv_heads": nkv, "head_dim": d, "intermediate": I, "vocab": V,
                   "prompt_len": args.prompt_len, "new_tokens": 1 + W + K_steps, "kv_block": 16, "cuda_graphs": True,
                   "l2": "inputs>L2: each step streams the weights", "peaks": pk["source"],
                   "model_write_s": round(write_s, 1), "model_gb": round(gb, 2)},
        "clocks": clock_info,
        # the reference is timed through its public API already (tokens counted as its result queue
        # delivers them), so this is the end-to-end figure too
        "e2e": {"value": r["tok_s"], "unit": "tok/s", "steps": K_steps, "h2d_bytes_per_step": None,
                "d2h_bytes_per_step": args.batch * 4},
        "gpu_launches": 0,
        "reference": {"decode_tokens_timed": r["decode_tokens_timed"], "requests_ended_early": r["requests_ended_early"],
                      "load_seconds": r["load_seconds"], "total_seconds": r["total_seconds"]},
    }
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=96)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill measurement")
    ap.add_argument("--no-decode", action="store_true", help="prefill measurement only (for profiling)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="model shape (default: the metric's 8b)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from firefly_b200.engine.engine import Engine, EngineOptions
    from firefly_b200.engine.loading import random_model
    from firefly_b200.engine.request import GenerationRequest
    from firefly_b200.engine.runner import StepEntry
    from firefly_b200.models import config_from_dict
    from firefly_b200.ops import kernels as K
    from firefly_b200.sampling import SamplingParams

    shape = load_shape(args.shape)
    full_layers = shape["num_hidden_layers"]
    if args.layers:
        shape["num_hidden_layers"] = args.layers
    # room for the prompt and every decode step of the run (a long --steps grows the context)
    need_ctx = args.prompt_len + 1 + args.warmup + 2 * args.steps + 6 + max(args.batch, 64)
    args.context = max(args.context, need_ctx)
    shape["max_position_embeddings"] = max(shape["max_position_embeddings"], args.context)
    cfg = config_from_dict(shape)
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    pk = peaks()
    es = 2 if args.dtype == "bfloat16" else 4

    t0 = time.time()
    model = random_model(cfg, seed=0, dtype=args.dtype, device=dev)
    torch.cuda.synchronize()
    build_s = time.time() - t0

    L, H, I, V = cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    nq, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    layer_params = (nq + 2 * nkv) * d * H + nq * d * H + 3 * H * I
    weight_bytes = (L * layer_params + V * H) * es + (2 * L + 1) * H * 4
    kv_bytes_per_token = L * 2 * nkv * d * es
    P = args.prompt_len
    K_steps, W = args.steps, args.warmup
    need_new = 1 + W + 2 * K_steps + 6
    gen = torch.Generator().manual_seed(1234)

    def make_engine(B, steps=None):
        # pages for what this engine's requests will hold, not for the whole context
        ctx = args.context if steps is None else min(args.context, P + 1 + W + 2 * steps + 6 + max(B, 64))
        opts = EngineOptions(max_prefill_chunk_size=P, max_batch_size_limit=max(B, 1),
                             max_num_batched_tokens=max(P, B), kv_block_size=16,
                             num_kv_blocks=B * (-(-ctx // 16)),      # max_model_len: the configuration's
                             eos_token_ids=[], graph_batch_sizes=(1, 2, 4, 8, 16, 32, 64))
        return Engine(model, cfg, options=opts)

    def start_requests(eng, B):
        reqs = []
        for i in range(B):
            ids = torch.randint(0, V, (P,), generator=gen).tolist()
            r = GenerationRequest(f"b{i}", ids, SamplingParams(max_tokens=max(256, need_new + B), ignore_eos=True))   # early requests decode while later prompts come in
            eng.add_request(r)
            reqs.append(r)
        while any(len(r.generated_tokens) == 0 for r in reqs):   # prompts in, first token sampled
            eng.step()
        return reqs

    def device_timed_decode(eng, reqs, steps):
        """``steps`` decode steps back to back on the device.  Returns (ms, own kernel launches)."""
        g = eng.graphs
        n = len(reqs)
        b = g._bucket_for(n)
        lay = b.layout
        for r in reqs:
            assert eng.cache.grow(r.cache, r.cache.num_tokens + steps + 1)
        entries = [StepEntry(r.cache, [r.generated_tokens[-1]], [0]) for r in reqs]
        # every step's metadata is made beforehand and parked on the device: the head of the buffer
        # (tokens, positions, lengths, table updates) per step; the block tables themselves, which
        # hold all the pages of the run already, go up once in front of the timed region
        head = lay.head_size
        staged_h = torch.empty((steps, head), dtype=torch.int32).pin_memory()
        base = [r.cache.num_tokens for r in reqs]
        for s in range(steps):
            for r, c in zip(reqs, base):
                r.cache.num_tokens = c + s          # positions of this step
            g._fill(b, entries)
            if not g._write_updates(b):
                assert s == 0, "only the first step may change more table entries than the update list holds"
                b.meta_dev.copy_(b.meta_host)
            staged_h[s].copy_(b.meta_host[:head])
        for r, c in zip(reqs, base):
            r.cache.num_tokens = c
        staged = staged_h.to(dev, non_blocking=True)
        toks = torch.empty((steps, n), dtype=torch.int32, device=dev)
        # the graph the engine itself would replay for these requests
        graph, launches = b.graph, b.launches
        if b.by_length is not None and K.lengths_differ_much(base):
            graph, launches = b.by_length[0], b.by_length[2]
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        ev0.record()
        for s in range(steps):
            b.meta_dev[:head].copy_(staged[s], non_blocking=True)
            if s:
                b.meta_dev[lay.token_ids: lay.token_ids + n].copy_(toks[s - 1], non_blocking=True)
            graph.replay()
            toks[s].copy_(b.tokens[:n], non_blocking=True)
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1)
        host = toks.cpu().tolist()
        for s in range(steps):                      # keep the engine's books right
            for r, t in zip(reqs, host[s]):
                eng.cache.advance(r.cache, 1)
                eng.scheduler.append_token(r, t)
        return ms, steps * launches

    def e2e_decode(eng, reqs, steps):
        n = len(reqs)
        torch.cuda.synchronize()
        h2d0, replays0 = eng.graphs.h2d_bytes, eng.graphs.replays
        t = time.perf_counter()
        produced = 0
        for _ in range(steps):
            outs = eng.step()
            assert len(outs) == n
            produced += len(outs)
        produced += len(eng.drain())                # a step launched ahead belongs to the timed work
        torch.cuda.synchronize()
        dt = time.perf_counter() - t
        # bytes of metadata the replays of this region uploaded (counted from the copies), per replay;
        # tokens and the status word come back
        h2d = (eng.graphs.h2d_bytes - h2d0) / max(1, eng.graphs.replays - replays0)
        return dt, produced, h2d, n * 4 + 4

    def decode_point(B, steps, with_e2e):
        eng = make_engine(B, steps)
        reqs = start_requests(eng, B)
        for _ in range(W):
            eng.step()
        eng.drain()
        assert eng.stats["graph_steps"] >= W, "decode did not run from CUDA graphs"
        # The step time drifts upward by a few per cent over the first hundreds of steps at full
        # power, so the end-to-end steps are split: half before the device-timed bracket, half after.
        e2e_dt = e2e_produced = 0
        if with_e2e:
            e2e_dt, e2e_produced, h2d, d2h = e2e_decode(eng, reqs, steps // 2)
        ctx0 = reqs[0].cache.num_tokens
        ms, launches = device_timed_decode(eng, reqs, steps)
        res = {"B": B, "ms_per_step": ms / steps, "tok_s": B * steps / (ms / 1e3), "launches": launches,
               "ctx_mean": ctx0 + steps / 2}
        if with_e2e:
            dt, produced, h2d, d2h = e2e_decode(eng, reqs, steps - steps // 2)
            dt, produced = dt + e2e_dt, produced + e2e_produced
            res["e2e"] = {"value": produced / dt, "unit": "tok/s", "steps": steps,
                          "steps_launched_ahead": eng.stats["launched_ahead"], "h2d_bytes_per_step": h2d,
                          "d2h_bytes_per_step": d2h}
        eng.runner.check_status()
        del eng
        torch.cuda.empty_cache()
        return res

    def prefill_point():
        eng = make_engine(1)
        times = []
        for it in range(3 + 5):
            ids = torch.randint(0, V, (P,), generator=gen).tolist()
            rc = eng.cache.admit(f"p{it}")
            assert eng.cache.grow(rc, P)
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            ev0.record()
            eng.runner.step([StepEntry(rc, ids, [P - 1])])
            ev1.record()
            torch.cuda.synchronize()
            if it >= 3:
                times.append(ev0.elapsed_time(ev1))
            eng.cache.free(rc)
        eng.runner.check_status()
        del eng
        torch.cuda.empty_cache()
        ms = statistics.median(times)
        flops = 2.0 * P * L * layer_params + 2.0 * V * H + L * 4.0 * nq * d * (P * (P + 1) / 2)
        return {"value": P / (ms / 1e3), "tokens": P, "ms": ms,
                "frac": flops / (ms / 1e3) / (pk["bf16_tflops_sustained" if False else "bf16_tflops"] * 1e12),
                "tflops": flops / (ms / 1e3) / 1e12}

    def prefill_chunked_point(chunk=256):
        """The prompt of P tokens fed through ``Engine.step`` in portions of ``chunk`` tokens (256: the
        reference's --max-prefill-chunk-size; None: the engine's default, which does not cut a prompt
        while no request is decoding): wall time from the first step to the first sampled token on the
        host, median of five prompts."""
        opts = EngineOptions(max_prefill_chunk_size=chunk, max_batch_size_limit=1, max_num_batched_tokens=8192,
                             kv_block_size=16, num_kv_blocks=-(-(P + 64) // 16), eos_token_ids=[])
        eng = Engine(model, cfg, options=opts)
        times = []
        for it in range(2 + 5):
            ids = torch.randint(0, V, (P,), generator=gen).tolist()
            req = GenerationRequest(f"c{it}", ids, SamplingParams(max_tokens=1, ignore_eos=True))
            eng.add_request(req)
            torch.cuda.synchronize()
            t = time.perf_counter()
            steps = 0
            while eng.has_unfinished_requests():
                eng.step()
                steps += 1
            torch.cuda.synchronize()
            if it >= 2:
                times.append((time.perf_counter() - t) * 1e3)
        eng.runner.check_status()
        del eng
        torch.cuda.empty_cache()
        ms = statistics.median(times)
        return {"value": P / (ms / 1e3), "tokens": P, "chunk": chunk, "steps": steps, "ms": ms}

    if args.no_decode:
        print(json.dumps({"prefill": prefill_point(), "prefill_chunked": prefill_chunked_point(),
                          "prefill_engine_default": prefill_chunked_point(None), "config": {"layers": L}}))
        return 0
    clocks = ClockSampler()
    if not os.environ.get("FF_NO_CLOCKS"):
        clocks.start()
    main_res = decode_point(args.batch, K_steps, with_e2e=True)
    clock_info = clocks.stop()
    prefill = None if args.no_prefill else prefill_point()
    prefill_chunked = None if args.no_prefill else prefill_chunked_point()
    if prefill_chunked is not None:
        by_default = prefill_chunked_point(None)
        prefill_chunked["engine_default_ms"] = by_default["ms"]
        prefill_chunked["engine_default_steps"] = by_default["steps"]
    points = {}
    if not args.no_points:
        for B in (1, 64):
            r = decode_point(B, min(K_steps, 64), with_e2e=False)
            points[f"decode_b{B}"] = r["tok_s"]
            points[f"decode_b{B}_ms_per_step"] = r["ms_per_step"]

    step_bytes = weight_bytes + args.batch * main_res["ctx_mean"] * kv_bytes_per_token
    achieved = step_bytes / (main_res["ms_per_step"] / 1e3) / 1e9
    out = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-{args.shape.upper()}-shaped {args.dtype}, {P}-token prompts)",
        "value": main_res["tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": K_steps, "warmup": W,
        "ms_per_step": main_res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic",
        "impl": "ours",
        "config": {"model": f"Qwen3-{args.shape.upper()}-shaped random weights", "global_batch": args.batch, "seq_len": args.context,
                   "parallelism": "single GPU", "layers": L, "layers_of_config": full_layers, "hidden": H,
                   "q_heads": nq, "kv_heads": nkv, "head_dim": d, "intermediate": I, "vocab": V,
                   "prompt_len": P, "new_tokens": need_new, "kv_block": 16, "cuda_graphs": True,
                   "max_positions": cfg.max_position_embeddings,
                   "l2": (f"inputs>L2: each step streams {step_bytes / 1e9:.1f} GB of weights, keys and values"
                          if step_bytes > 2 * 126e6 else
                          f"step reads {step_bytes / 1e6:.0f} MB, not larger than L2; no flush between steps"),
                   "peaks": pk["source"], "model_build_s": round(build_s, 1)},
        "clocks": clock_info,
        "e2e": main_res["e2e"],
        "gpu_launches": main_res["launches"],
        "prefill": prefill,
        "prefill_chunked": prefill_chunked,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
