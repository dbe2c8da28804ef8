#!/usr/bin/env python3
"""Records what the reference's scheduler decides, for tests/test_scheduler.py to compare with.

The reference's model code cannot be built here (CUDA-only FP16, network-fetched dependencies), but
its scheduler and radix tree are plain host C++: this script compiles ``src/scheduler.cc`` and
``src/radix_tree.cc`` of a checkout of the reference, unchanged, together with the driver
``ref_scheduler_trace.cc`` beside this file, runs the scenarios below and writes
``ref_scheduler_trace.json``.  Scenarios are kept to what the reference does soundly: distinct
prompts (nothing shared through its radix tree), enough pages (it neither preempts nor frees), pages
of 16 tokens (fixed there).

    python tests/golden/make_ref_scheduler_golden.py /path/to/firefly
"""
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))

# name -> (pages, most active requests, max_prefill_chunk_size, [(id, prompt length, max_tokens), ...])
SCENARIOS = {
    "three_requests_chunk_17": (64, 64, 17, [("a", 40, 4), ("b", 5, 3), ("c", 23, 5)]),
    "chunk_256_default": (64, 64, 256, [("a", 300, 2), ("b", 16, 3), ("c", 1, 4), ("d", 257, 1)]),
    "two_active_at_most": (64, 2, 8, [("a", 20, 2), ("b", 3, 6), ("c", 9, 2), ("d", 8, 1)]),
}


def main() -> int:
    if len(sys.argv) != 2:
        print(__doc__, file=sys.stderr)
        return 2
    ref = sys.argv[1]
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "ref_sched")
        subprocess.run(["g++", "-std=c++23", "-O1", "-I", os.path.join(ref, "include"),
                        os.path.join(HERE, "ref_scheduler_trace.cc"), os.path.join(ref, "src", "scheduler.cc"),
                        os.path.join(ref, "src", "radix_tree.cc"), "-o", exe], check=True)
        for name, (pages, limit, chunk, reqs) in SCENARIOS.items():
            args = [exe, str(pages), str(limit), str(chunk)]
            for rid, n, m in reqs:
                args += [rid, str(n), str(m)]
            steps = json.loads(subprocess.run(args, check=True, capture_output=True, text=True).stdout)
            out[name] = {"pages": pages, "max_batch_size_limit": limit, "max_prefill_chunk_size": chunk,
                         "requests": [list(r) for r in reqs],
                         # per iteration: [request, tokens in the cache before, tokens fed, pages held]
                         "steps": steps}
    with open(os.path.join(HERE, "ref_scheduler_trace.json"), "w") as fh:
        json.dump(out, fh, indent=1)
        fh.write("\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
