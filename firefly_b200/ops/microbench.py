"""Timing single kernels and single steps on the device, for the figures under ``profiles/``.

    python -m firefly_b200.ops.microbench gemm  [--tokens 128,256,512] [--shape 8b]
        the package's matrix products alone against the library's, at a model's layer shapes
    python -m firefly_b200.ops.microbench step  [--tokens 96,128,256,512] [--shape 8b] [--layers N] [--pair]
        one step of a prompt portion of that many tokens (context 1024): queued by the host launch by
        launch, and replayed from a CUDA graph

    python -m firefly_b200.ops.microbench timeline [--tokens 2048] [--context 0] [--batch 1] [--layers 4] [--shape 8b]
        the kernels of one replayed step in order with their device times (a CUPTI timeline through
        torch.profiler): ``--batch`` requests with ``--tokens`` new tokens each behind ``--context`` tokens

    python -m firefly_b200.ops.microbench load [--shape 8b]
        a bfloat16 model folder of that shape written to a temporary folder, then loaded twice through
        the engine's loader: seconds, GB/s, the arena's size and the peak of device memory

CUDA events around 20 (gemm) or 40 (step) repetitions after warm-up; weights are rotated through more
than 400 MB in the gemm case so that they come from HBM, not from L2.
"""
from __future__ import annotations

import argparse
import time

import torch

from . import kernels as K

SHAPES = {   # hidden, intermediate, q heads, kv heads, head size, layers, vocabulary
    "8b": (4096, 12288, 32, 8, 128, 36, 151936),
    "0.6b": (1024, 3072, 16, 8, 128, 28, 151936),
    "32b": (5120, 25600, 64, 8, 128, 64, 151936),
}


def _time(fn, n):
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n * 1000.0          # microseconds


def gemm(args) -> None:
    H, I, nq, nkv, d, _, _ = SHAPES[args.shape]
    shapes = {"qkv": ((nq + 2 * nkv) * d, H), "o": (H, nq * d), "gate_up": (2 * I, H), "down": (H, I)}
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    K.set_exact_matmul()
    for name, (N, Kd) in shapes.items():
        copies = max(2, int(400e6 // (N * Kd * 2)) + 1)
        ws = [torch.randn(N, Kd, device="cuda").to(torch.bfloat16) for _ in range(copies)]
        for T in args.tokens:
            x = torch.randn(T, Kd, device="cuda").to(torch.bfloat16)
            out = torch.empty(T, N, dtype=torch.bfloat16, device="cuda")
            lib = _time(lambda i: torch.mm(x, ws[i % copies].t(), out=out), 20)
            line = f"{name:8s} {N:6d} x {Kd:5d}  T={T:4d}  library {lib:6.1f} us ({N * Kd * 2 / lib / 1e6:4.2f} TB/s)"
            if T <= 256:
                for s in (1, 4, 8):
                    t = _time(lambda i: K.gemm_tc(x, ws[i % copies], out, K.EPI_BF16, s, status), 20)
                    line += f" | one-block s{s} {t:6.1f}"
            for r in (1, 2, 3):
                if K.gemm_pair_plan(T, N, Kd, r)[1] != r:
                    continue
                t = _time(lambda i: K.gemm_pair(x, ws[i % copies], out, K.EPI_BF16, r, status), 20)
                line += f" | pair r{r} {t:6.1f}"
            print(line, flush=True)
        del ws
    print("status", int(status))


def step(args) -> None:
    from ..config.qwen3 import Qwen3Config
    from ..engine.engine import Engine, EngineOptions
    from ..engine.loading import random_model
    from ..engine.runner import StepEntry
    H, I, nq, nkv, d, L, V = SHAPES[args.shape]
    cfg = Qwen3Config.from_dict(dict(
        architectures=["Qwen3ForCausalLM"], hidden_size=H, intermediate_size=I, num_hidden_layers=args.layers or L,
        num_attention_heads=nq, num_key_value_heads=nkv, head_dim=d, vocab_size=V, max_position_embeddings=8192,
        rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=args.shape == "0.6b"))
    K.USE_PAIR_GEMM = bool(args.pair)
    model = random_model(cfg, 0)
    ids = torch.randint(0, V, (4096,), generator=torch.Generator().manual_seed(0)).tolist()
    for T in args.tokens:
        eng = Engine(model, cfg, options=EngineOptions(max_prefill_chunk_size=T, num_kv_blocks=512, max_batch_size_limit=2,
                                                       use_cuda_graphs=False))
        rc = eng.cache.admit("r")
        p = 0
        while p < 1024:
            assert eng.cache.grow(rc, p + T)
            eng.runner.step([StepEntry(rc, ids[p:p + T], [])])
            p += T
        assert eng.cache.grow(rc, p + T)
        ctx = eng.runner.build_context([StepEntry(rc, ids[p:p + T], [])])
        for _ in range(2):
            model.forward(ctx)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(5):
            model.forward(ctx)
        e1.record()
        host = (time.perf_counter() - t0) / 5 * 1e3
        torch.cuda.synchronize()
        eager = e0.elapsed_time(e1) / 5
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            model.forward(ctx)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            model.forward(ctx)
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(40):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        eng.runner.check_status()
        print(f"{args.shape} {cfg.num_hidden_layers} layers, {T} tokens behind 1024: launch by launch {eager:.3f} ms "
              f"(the host needs {host:.3f} ms to queue it), graph replay {e0.elapsed_time(e1) / 40:.3f} ms", flush=True)
        del eng, graph


def timeline(args) -> None:
    """One step replayed from a CUDA graph under the profiler.  With programmatic dependent launch a
    kernel's recorded start lies before its real work, so beside each kernel's own time the step from
    the end of the kernel before to its own end is printed: those add up to the step."""
    import collections
    from torch.profiler import ProfilerActivity, profile
    from ..config.qwen3 import Qwen3Config
    from ..engine.engine import Engine, EngineOptions
    from ..engine.loading import random_model
    from ..engine.runner import StepEntry
    H, I, nq, nkv, d, L, V = SHAPES[args.shape]
    layers = args.layers or 4
    cfg = Qwen3Config.from_dict(dict(
        architectures=["Qwen3ForCausalLM"], hidden_size=H, intermediate_size=I, num_hidden_layers=layers,
        num_attention_heads=nq, num_key_value_heads=nkv, head_dim=d, vocab_size=V, max_position_embeddings=40960,
        rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=args.shape == "0.6b"))
    model = random_model(cfg, 0)
    T, B, C = args.tokens[0], args.batch, args.context
    ids = torch.randint(0, V, (C + T,), generator=torch.Generator().manual_seed(0)).tolist()
    eng = Engine(model, cfg, options=EngineOptions(
        max_prefill_chunk_size=max(T, C, 1), max_num_batched_tokens=max(B * T, C, 1), max_batch_size_limit=max(B, 1),
        num_kv_blocks=B * (-(-(C + T) // 16) + 1) + 8, max_model_len=C + T + 16, use_cuda_graphs=False))
    caches = []
    for r in range(B):
        rc = eng.cache.admit(f"r{r}")
        if C:
            assert eng.cache.grow(rc, C)
            eng.runner.step([StepEntry(rc, ids[:C], [])])
        assert eng.cache.grow(rc, C + T)
        caches.append(rc)
    ctx = eng.runner.build_context([StepEntry(rc, ids[C:C + T], [T - 1]) for rc in caches])
    for _ in range(2):
        model.forward(ctx)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        model.forward(ctx)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        model.forward(ctx)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    print(f"{args.shape}, {layers} layers, {B} x {T} tokens behind {C}: {e0.elapsed_time(e1) / 20 * 1000:.1f} us a replayed step")
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        graph.replay()
        torch.cuda.synchronize()
    evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                 key=lambda e: e.time_range.start)
    eng.runner.check_status()
    total = collections.OrderedDict()
    prev_end = None
    print("   step us   own us  kernel (in launch order)")
    for e in evs:
        own = e.time_range.end - e.time_range.start
        step_us = e.time_range.end - (prev_end if prev_end is not None else e.time_range.start)
        prev_end = max(prev_end or 0, e.time_range.end)
        print(f"  {step_us:8.1f} {own:8.1f}  {e.name[:100]}")
        t = total.setdefault(e.name[:100], [0, 0.0])
        t[0] += 1
        t[1] += step_us
    print("sums by kernel:")
    for name, (n, us) in sorted(total.items(), key=lambda kv: -kv[1][1]):
        print(f"  {us:9.1f} us  {n:4d} x  {name}")


def load(args) -> None:
    import json
    import os
    import shutil
    import struct
    import tempfile
    from ..config.qwen3 import Qwen3Config
    from ..engine.loading import load_model, random_model
    from ..models import expected_weights, spec_for
    H, I, nq, nkv, d, L, V = SHAPES[args.shape]
    cfg = Qwen3Config.from_dict(dict(
        architectures=["Qwen3ForCausalLM"], hidden_size=H, intermediate_size=I, num_hidden_layers=args.layers or L,
        num_attention_heads=nq, num_key_value_heads=nkv, head_dim=d, vocab_size=V, max_position_embeddings=40960,
        rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=args.shape == "0.6b"))
    folder = tempfile.mkdtemp(prefix="firefly_b200_load_")
    try:
        specs = [w for w in expected_weights(spec_for(cfg)) if not w.optional]
        header, off = {}, 0
        for w in specs:
            n = 2
            for x in w.shape:
                n *= x
            header[w.name] = {"dtype": "BF16", "shape": list(w.shape), "data_offsets": [off, off + n]}
            off += n
        blob = json.dumps(header, separators=(",", ":")).encode()
        blob += b" " * ((8 - len(blob) % 8) % 8)
        g = torch.Generator(device="cuda").manual_seed(0)
        with open(os.path.join(folder, "model.safetensors"), "wb") as fh:
            fh.write(struct.pack("<Q", len(blob)))
            fh.write(blob)
            for w in specs:
                x = torch.randn(w.shape, generator=g, device="cuda", dtype=torch.float32)
                x = (1 + 0.01 * x) if len(w.shape) == 1 else 0.02 * x
                fh.write(x.to(torch.bfloat16).view(torch.int16).cpu().numpy().tobytes())
        with open(os.path.join(folder, "config.json"), "w") as fh:
            json.dump(cfg.to_dict(), fh)
        del x
        torch.cuda.empty_cache()
        torch.cuda.synchronize()
        print(f"{args.shape}: a folder of {off / 1e9:.1f} GB", flush=True)
        for attempt in ("first load (the file is in the page cache)", "second load"):
            torch.cuda.reset_peak_memory_stats()
            base = torch.cuda.memory_allocated()
            t0 = time.perf_counter()
            model, _ = load_model(folder, dtype="bfloat16")
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            f = model.load_facts
            print(f"{args.shape} {attempt}: {dt:.2f} s ({f['file_bytes'] / dt / 1e9:.1f} GB/s), arena "
                  f"{f['arena_bytes'] / 1e9:.2f} GB, peak device memory "
                  f"{(torch.cuda.max_memory_allocated() - base) / 1e9:.2f} GB, files registered with the driver "
                  f"{f['pinned_files']} of {f['files']}", flush=True)
            del model
            torch.cuda.empty_cache()
        t0 = time.perf_counter()
        model = random_model(cfg, 0)
        torch.cuda.synchronize()
        print(f"{args.shape} random weights drawn on the device: {time.perf_counter() - t0:.2f} s")
    finally:
        shutil.rmtree(folder, ignore_errors=True)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m firefly_b200.ops.microbench")
    ap.add_argument("what", choices=["gemm", "step", "timeline", "load"])
    ap.add_argument("--tokens", default=None)
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES))
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--context", type=int, default=0, help="timeline: tokens already in the cache")
    ap.add_argument("--batch", type=int, default=1, help="timeline: requests in the step")
    ap.add_argument("--pair", action="store_true", help="route products of 65 to 512 tokens to the two-SM kernel")
    args = ap.parse_args(argv)
    default = {"gemm": "128,256,512", "step": "96,128,256,512", "timeline": "2048", "load": "0"}[args.what]
    args.tokens = [int(t) for t in (args.tokens or default).split(",")]
    if not torch.cuda.is_available():
        print("microbench: needs a CUDA device")
        return 1
    {"gemm": gemm, "step": step, "timeline": timeline, "load": load}[args.what](args)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
