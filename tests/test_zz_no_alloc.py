"""The allocation-free decode attention, called through its exported C symbol.

Some hosts of these kernels cannot allocate device memory when they call: they
gave all of it to their own pool at start-up, or they cannot afford the
device-wide synchronisation an allocation brings.  ``ff_attn_decode_static`` keeps
the split-KV scratch in an array inside the library; here it must give what the
regular entry point gives, on two calls in a row that share that array.  The file
sorts last so that a run that stops at the first failure has run everything else.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

from test_kernels_gpu import _attention_case

pytestmark = pytest.mark.gpu


def _ptr(t):
    return c_void_p(t.data_ptr())


def test_static_scratch_entry_matches_regular_entry_twice():
    from firefly_b200.ops import kernels as K
    from firefly_b200.ops.build import load_module
    d, nq, nkv, block = 128, 8, 2, 16
    lib = load_module("attention_decode_static.cu", {"FF_HEAD_DIM": d})
    fn = lib.ff_attn_decode_static
    fn.restype = c_int
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (seqs, splits, window, seed) in enumerate([
            ([(0, 1), (63, 1), (200, 1), (517, 1), (64, 1)], 5, 0, 1),
            ([(300, 1), (5, 1), (129, 1)], 3, 100, 2)]):       # fewer splits: stale entries stay behind
        c = _attention_case(d, nq, nkv, block, seqs, window or None, torch.bfloat16, seed=seed)
        n = len(seqs)
        dev = {k: c[k].to("cuda") for k in ("q", "pages", "table", "cu_q", "ctx_lens")}
        want = torch.zeros(c["q"].shape, dtype=torch.bfloat16, device="cuda")
        part_o = torch.empty(n * nq * splits * d, device="cuda")
        part_ml = torch.empty(n * nq * splits * 2, device="cuda")
        K.attn_decode(dev["q"], nq * d, dev["pages"], dev["table"], dev["cu_q"], dev["ctx_lens"], n, want,
                      part_o, part_ml, nq, nkv, d, 1 / math.sqrt(d), window, splits)
        got = torch.zeros_like(want)
        # the driver's own count of free bytes sees every allocation on the device, also one that
        # bypasses torch's allocator.  It is held on the second call: at the first one the driver may
        # still be loading the library's module (its code and the fixed array itself, 2 MB)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()
        rc = fn(_ptr(dev["q"]), c_int(nq * d), _ptr(dev["pages"]), _ptr(dev["table"]),
                c_int(dev["table"].shape[1]), _ptr(dev["cu_q"]), _ptr(dev["ctx_lens"]), c_int(n), _ptr(got),
                c_int(nq * d), c_int(nq), c_int(nkv), c_int(block), c_int(dev["pages"].shape[0]),
                c_float(1 / math.sqrt(d)), c_int(window), c_int(splits), stream)
        assert rc == 0, f"call {call}: return code {rc}"
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        free_after, _ = torch.cuda.mem_get_info()
        if call > 0:
            assert free_after >= free_before, f"call {call}: {free_before - free_after} bytes of device memory were taken"
        ref = c["want"]
        scale = float(ref.abs().max())
        assert float((got.cpu().double() - want.cpu().double()).abs().max()) <= 2e-2 * scale
        assert float((got.cpu().double() - ref).abs().max()) <= 2e-2 * scale
    # beyond the built-in array: refused, nothing launched
    rc = fn(_ptr(dev["q"]), c_int(nq * d), _ptr(dev["pages"]), _ptr(dev["table"]),
            c_int(dev["table"].shape[1]), _ptr(dev["cu_q"]), _ptr(dev["ctx_lens"]), c_int(3), _ptr(got),
            c_int(nq * d), c_int(nq), c_int(nkv), c_int(block), c_int(dev["pages"].shape[0]),
            c_float(1 / math.sqrt(d)), c_int(0), c_int(4096), stream)
    assert rc == -3
