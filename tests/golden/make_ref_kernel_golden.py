#!/usr/bin/env python3
"""Records what the reference's own CUDA kernels compute, for tests/test_ref_kernel_golden.py.

The reference's kernel sources (``src/kernels/{norm,rope,activation,embedding,add,sampling,
attention}.cu``) are compiled unchanged, with the reference's own compiler options
(``--use_fast_math``, C++20; cmake/CUDAConf.cmake:5-17), behind two stand-ins beside this file:
``ref_shim/mdspan/mdspan.hpp`` (the mdspan header the reference fetches at build time, mapped to the
CUDA toolkit's) and ``ref_shim/tensor_shim.cu`` (the members of ``Tensor`` that the launchers use,
over caller-owned memory, and a C interface over ``firefly::kernels::*``).  Nothing of this
package is involved.  The cases are ones the reference's kernels support: FP16, head size 128, rows
that are multiples of 8, cache pages of 16 tokens, one query token per sequence for the attention
(its decode branch, ``paged_attention_kernel``, src/kernels/attention.cu:291-447).  The prefill
branch (``flash_attn_wmma_kernel``) is left out: it reads rows past the sequence's end and scales
accumulator elements by other rows' factors (src/kernels/attention.cu:78,94-98,212-215,240).

Inputs are drawn on the CPU from the seeds in ``CASES``; only the outputs are stored.

    python tests/golden/make_ref_kernel_golden.py build /path/to/firefly OUT.so     (needs nvcc)
    python tests/golden/make_ref_kernel_golden.py run OUT.so [GOLDEN.npz]          (needs a GPU)
"""
import ctypes
import os
import subprocess
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "ref_kernels_golden.npz")
KERNEL_FILES = ("norm", "rope", "activation", "embedding", "add", "sampling", "attention")


def half(gen, *shape, scale=1.0):
    return (torch.randn(*shape, generator=gen, dtype=torch.float32) * scale).to(torch.float16)


def cases():
    """name -> dict of CPU inputs (FP16 / int32 tensors and plain numbers)."""
    out = {}
    g = torch.Generator().manual_seed(101)
    out["rms_norm_rows"] = dict(x=half(g, 5, 256, scale=3.0), w=1 + half(g, 256, scale=0.1), eps=1e-6)
    g = torch.Generator().manual_seed(102)
    out["rms_norm_heads"] = dict(x=half(g, 24, 128), w=1 + half(g, 128, scale=0.1), eps=1e-5)
    g = torch.Generator().manual_seed(103)
    out["rope_theta1e6"] = dict(q=half(g, 2, 3, 4, 128), k=half(g, 2, 3, 2, 128), theta=1e6,
                                context_lens=torch.tensor([0, 37], dtype=torch.int32))
    g = torch.Generator().manual_seed(104)
    out["rope_theta1e4"] = dict(q=half(g, 1, 5, 2, 128), k=half(g, 1, 5, 2, 128), theta=1e4,
                                context_lens=torch.tensor([11], dtype=torch.int32))
    g = torch.Generator().manual_seed(105)
    out["swiglu"] = dict(gate=half(g, 4, 64, scale=3.0), up=half(g, 4, 64))
    g = torch.Generator().manual_seed(106)
    out["add"] = dict(x=half(g, 3, 40), y=half(g, 3, 40))
    g = torch.Generator().manual_seed(107)
    out["embedding"] = dict(ids=torch.tensor([[3, 49, 0], [17, 3, 48]], dtype=torch.int32), table=half(g, 50, 64))
    g = torch.Generator().manual_seed(108)
    logits = half(g, 3, 1000, scale=2.0)
    logits[1, 700] = logits[1, 123] = 9.0          # a tie: which index wins is the reference's choice
    logits[2, 999] = 11.0
    out["argmax"] = dict(logits=logits)
    g = torch.Generator().manual_seed(109)
    nq, nkv, d, blocks = 8, 2, 128, 8
    ctx = [0, 20, 45]                               # keys 0..ctx are read (ctx + 1 of them)
    table = torch.full((3, 3), 0, dtype=torch.int32)
    table[0, :1] = torch.tensor([5])
    table[1, :2] = torch.tensor([2, 7])
    table[2, :3] = torch.tensor([6, 0, 3])
    kc, vc = half(g, blocks, 16, nkv, d), half(g, blocks, 16, nkv, d)
    q = half(g, 3, 1, nq, d)
    q[2, 0, 5] *= 6.0                               # one head with a sharp softmax
    out["paged_attention"] = dict(q=q, k_cache=kc, v_cache=vc, table=table,
                                  context_lens=torch.tensor(ctx, dtype=torch.int32), nq=nq, nkv=nkv, d=d)
    return out


def build(reference: str, out_lib: str) -> None:
    srcs = [os.path.join(reference, "src", "kernels", f + ".cu") for f in KERNEL_FILES]
    cmd = ["nvcc", "-std=c++20", "--use_fast_math", "--expt-relaxed-constexpr", "-gencode",
           "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC",
           "-I", os.path.join(reference, "include"), "-I", os.path.join(HERE, "ref_shim"), "-o", out_lib,
           *srcs, os.path.join(HERE, "ref_shim", "tensor_shim.cu")]
    subprocess.run(cmd, check=True)


def run(lib_path: str, out_path: str = GOLDEN) -> None:
    lib = ctypes.CDLL(lib_path)
    dev = torch.device("cuda:0")
    P = lambda t: ctypes.c_void_p(t.data_ptr())     # noqa: E731
    res = {}

    def ok(code, what):
        if code != 0:
            raise RuntimeError(f"{what}: code {code}")
    cs = cases()
    for name in ("rms_norm_rows", "rms_norm_heads"):
        c = cs[name]
        x, w = c["x"].to(dev), c["w"].to(dev)
        o = torch.empty_like(x)
        ok(lib.ref_rms_norm(P(x), P(w), P(o), x.shape[0], x.shape[1], ctypes.c_double(c["eps"])), name)
        res[name] = o.cpu().numpy()
    for name in ("rope_theta1e6", "rope_theta1e4"):
        c = cs[name]
        q, k, cl = c["q"].to(dev), c["k"].to(dev), c["context_lens"].to(dev)
        B, S, nq, d = q.shape
        ok(lib.ref_rope(P(q), P(k), B, S, nq, k.shape[2], d, ctypes.c_float(c["theta"]), P(cl)), name)
        res[name + ".q"], res[name + ".k"] = q.cpu().numpy(), k.cpu().numpy()
    c = cs["swiglu"]
    g_, u_ = c["gate"].to(dev), c["up"].to(dev)
    o = torch.empty_like(g_)
    ok(lib.ref_swiglu(P(g_), P(u_), P(o), g_.shape[0], g_.shape[1]), "swiglu")
    res["swiglu"] = o.cpu().numpy()
    c = cs["add"]
    x, y = c["x"].to(dev), c["y"].to(dev)
    ok(lib.ref_add_inplace(P(x), P(y), x.shape[0], x.shape[1]), "add")
    res["add"] = x.cpu().numpy()
    c = cs["embedding"]
    ids, table = c["ids"].to(dev), c["table"].to(dev)
    o = torch.empty((*ids.shape, table.shape[1]), dtype=torch.float16, device=dev)
    ok(lib.ref_embedding(P(ids), P(table), P(o), ids.shape[0], ids.shape[1], table.shape[0], table.shape[1]),
       "embedding")
    res["embedding"] = o.cpu().numpy()
    c = cs["argmax"]
    lg = c["logits"].to(dev)
    o = torch.empty(lg.shape[0], dtype=torch.int32, device=dev)
    ok(lib.ref_argmax(P(lg), P(o), lg.shape[0], lg.shape[1]), "argmax")
    res["argmax"] = o.cpu().numpy()
    c = cs["paged_attention"]
    q, kc, vc = c["q"].to(dev), c["k_cache"].to(dev), c["v_cache"].to(dev)
    tb, cl = c["table"].to(dev), c["context_lens"].to(dev)
    o = torch.empty((q.shape[0], 1, c["nq"] * c["d"]), dtype=torch.float16, device=dev)
    ok(lib.ref_paged_attention(P(q), P(kc), P(vc), P(o), P(tb), q.shape[0], c["nq"], c["nkv"], c["d"],
                               kc.shape[0], tb.shape[1], P(cl)), "paged_attention")
    res["paged_attention"] = o.cpu().numpy()
    np.savez_compressed(out_path, **res)
    print("wrote", out_path, {k: v.shape for k, v in res.items()})


if __name__ == "__main__":
    if len(sys.argv) == 4 and sys.argv[1] == "build":
        build(sys.argv[2], sys.argv[3])
    elif len(sys.argv) in (3, 4) and sys.argv[1] == "run":
        run(*sys.argv[2:])
    else:
        sys.exit(__doc__)
