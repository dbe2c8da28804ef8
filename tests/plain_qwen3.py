"""A plain, slow implementation of Qwen3 dense: whole sequences, no cache.

It is the oracle of the tests.  It shares no code with ``firefly_b200``: it takes
a plain dict of config.json keys and a dict ``{tensor name: torch tensor}``, runs
on the CPU in float64 (or any dtype asked for), and has one function per part.

It is written from the reference's formulas; each function cites the file and
lines whose arithmetic it restates.  The reference's engine as a whole cannot be
run here (CUDA-only FP16, a gRPC tool-chain fetched over the network, head size
128 only, no tied embeddings), but its kernels can be compiled unchanged behind a
small stand-in for its Tensor class: ``tests/golden/ref_kernels_golden.npz`` holds
what its RMSNorm, rotary, SwiGLU, residual-add, embedding, arg-max and decode
attention kernels computed on a B200, and ``tests/test_ref_kernel_golden.py``
holds the functions of this file to them.  Where the reference is wrong for a
general batch (prefill attention that ignores earlier portions,
src/model/qwen_model.cu:147-151 with the chunk-local mask of
src/kernels/attention.cu:173) this file follows the formula with absolute
positions.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """h[t,:] = E[id[t],:]  (src/kernels/embedding.cu:19-37)."""
    return table[ids.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w, the weight a plain multiplier
    (src/kernels/norm.cu:73-131)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * weight


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate-half rotary encoding over the whole head.

    x [T, heads, d]; for i in [0, d/2): f_i = theta^(-2i/d), a = pos * f_i,
    (x_i, x_{i+d/2}) <- (x_i cos a - x_{i+d/2} sin a, x_{i+d/2} cos a + x_i sin a)
    (src/kernels/rope.cu:68-95; position = context length + index, :34-35).
    """
    d = x.shape[-1]
    half = d // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / d)
    ang = positions.to(torch.float64)[:, None] * freq[None, :]          # [T, d/2]
    cos = torch.cos(ang).to(x.dtype)[:, None, :]
    sin = torch.sin(ang).to(x.dtype)[:, None, :]
    lo, hi = x[..., :half], x[..., half:]
    return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: Optional[float] = None,
              window: Optional[int] = None) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence.

    q [T, nq, d], k/v [T, nkv, d]; q head h uses kv head h // (nq/nkv)
    (src/kernels/attention.cu:44,304); scores (q.k)/sqrt(d) (:458), softmax over
    keys 0..t (the decode kernel's range, :320), output sum p_j v_j / l
    (:332-446).  ``window`` W keeps keys t-W+1..t only (not in the reference).
    """
    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    out = torch.empty_like(q)
    t = torch.arange(T)
    allowed = t[None, :] <= t[:, None]
    if window is not None:
        allowed &= t[None, :] > (t[:, None] - window)
    for h in range(nq):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, kh, :]
    return out


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """g / (1 + exp(-g)) * u  (src/kernels/activation.cu:15-19,76-80)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def swiglu_mlp(x, w_gate, w_up, w_down):
    """(silu(x Wg^T) * (x Wu^T)) Wd^T  (src/model/qwen_model.cu:164-174)."""
    return silu_mul(x @ w_gate.T, x @ w_up.T) @ w_down.T


def attention_block(x, w: Mapping[str, torch.Tensor], prefix: str, cfg: Mapping, positions,
                    *, window=None, kv_from: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
    """q,k,v projections, per-head q/k RMSNorm before the rotation, rotation,
    attention, output projection (src/model/qwen_model.cu:113-158).  Returns
    (output, (k, v)) so that another run may read this run's keys and values."""
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    T = x.shape[0]
    q = (x @ w[f"{prefix}.q_proj.weight"].T).view(T, nq, d)
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], cfg["rms_norm_eps"])
    q = rope(q, positions, cfg["rope_theta"])
    if kv_from is None:
        k = (x @ w[f"{prefix}.k_proj.weight"].T).view(T, nkv, d)
        v = (x @ w[f"{prefix}.v_proj.weight"].T).view(T, nkv, d)
        k = rms_norm(k, w[f"{prefix}.k_norm.weight"], cfg["rms_norm_eps"])
        k = rope(k, positions, cfg["rope_theta"])
    else:
        k, v = kv_from
    o = attention(q, k, v, window=window).reshape(T, nq * d)
    return o @ w[f"{prefix}.o_proj.weight"].T, (k, v)


def forward(cfg: Mapping, weights: Mapping[str, torch.Tensor], ids: Sequence[int], *,
            dtype: torch.dtype = torch.float64, windows: Optional[Sequence[Optional[int]]] = None,
            schedule: Optional[Sequence[Tuple[int, int, bool]]] = None) -> torch.Tensor:
    """Logits [T, vocab] at every position of one whole sequence.

    Pre-norm residual blocks (src/model/qwen_model.cu:106-175), final RMSNorm and
    output head (:177-188; the head is the embedding matrix when
    ``tie_word_embeddings``).  ``schedule`` lists runs (layer, cache slot, write);
    a run with write=False attends over the keys and values of the run that wrote
    its slot.  ``windows[layer]`` bounds that layer's attention.
    """
    w = {k: v.to(dtype) for k, v in weights.items()}
    L = cfg["num_hidden_layers"]
    ids_t = torch.as_tensor(list(ids), dtype=torch.long)
    T = ids_t.numel()
    positions = torch.arange(T)
    h = embedding(ids_t, w["model.embed_tokens.weight"])
    runs = schedule if schedule is not None else [(i, i, True) for i in range(L)]
    kv: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
    for layer, slot, write in runs:
        p = f"model.layers.{layer}"
        win = windows[layer] if windows is not None else None
        x = rms_norm(h, w[f"{p}.input_layernorm.weight"], cfg["rms_norm_eps"])
        a, new_kv = attention_block(x, w, f"{p}.self_attn", cfg, positions, window=win,
                                    kv_from=None if write else kv[slot])
        if write:
            kv[slot] = new_kv
        h = h + a
        x = rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        h = h + swiglu_mlp(x, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                           w[f"{p}.mlp.down_proj.weight"])
    x = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else w["lm_head.weight"]
    return x @ head.T


def greedy_pick(logits: torch.Tensor) -> int:
    """Index of the largest logit, the lowest such index on ties.  The reference's kernel keeps
    the lowest index within a thread by a strict '>' and leaves ties between threads to its block
    reduction (src/kernels/sampling.cu:27-37)."""
    top = logits.max()
    return int(torch.nonzero(logits == top)[0])


def greedy_generate(cfg, weights, prompt: Sequence[int], n_new: int, *, dtype=torch.float64) -> List[int]:
    """Arg-max decoding (lowest index on ties), recomputing the whole sequence
    each time (src/kernels/sampling.cu:27-37 for the arg-max)."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward(cfg, weights, ids, dtype=dtype)[-1]
        nxt = greedy_pick(logits)
        out.append(nxt)
        ids.append(nxt)
    return out


# --------------------------------------------------------------------------- #
# tiny configurations that differ in every size and option
# --------------------------------------------------------------------------- #
TINY_A = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              vocab_size=256, max_position_embeddings=128, rms_norm_eps=1e-6, rope_theta=10000.0,
              tie_word_embeddings=True)
TINY_B = dict(architectures=["Qwen3ForCausalLM"], hidden_size=96, intermediate_size=160,
              num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2, head_dim=32,
              vocab_size=384, max_position_embeddings=256, rms_norm_eps=1e-5, rope_theta=1000000.0,
              tie_word_embeddings=False)
# a third one with sizes that are no power of two anywhere, for the kernels' edges
TINY_C = dict(architectures=["Qwen3ForCausalLM"], hidden_size=72, intermediate_size=200,
              num_hidden_layers=2, num_attention_heads=3, num_key_value_heads=1, head_dim=48,
              vocab_size=333, max_position_embeddings=512, rms_norm_eps=3e-6, rope_theta=50000.0,
              tie_word_embeddings=False)


# head size 64: the size class of the tcgen05 attention kernel, with a group of 4
TINY_D = dict(architectures=["Qwen3ForCausalLM"], hidden_size=128, intermediate_size=272,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1, head_dim=64,
              vocab_size=500, max_position_embeddings=1024, rms_norm_eps=1e-6, rope_theta=10000.0,
              tie_word_embeddings=True)


def expected_tensor_shapes(cfg: Mapping) -> Dict[str, Tuple[int, ...]]:
    """Tensor names and shapes of a checkpoint (src/model/qwen_model.cu:58-92)."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    out = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,)}
    if not cfg.get("tie_word_embeddings", False):
        out["lm_head.weight"] = (V, H)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        out[f"{p}.input_layernorm.weight"] = (H,)
        out[f"{p}.post_attention_layernorm.weight"] = (H,)
        out[f"{p}.self_attn.q_proj.weight"] = (nq * d, H)
        out[f"{p}.self_attn.k_proj.weight"] = (nkv * d, H)
        out[f"{p}.self_attn.v_proj.weight"] = (nkv * d, H)
        out[f"{p}.self_attn.o_proj.weight"] = (H, nq * d)
        out[f"{p}.self_attn.q_norm.weight"] = (d,)
        out[f"{p}.self_attn.k_norm.weight"] = (d,)
        out[f"{p}.mlp.gate_proj.weight"] = (I, H)
        out[f"{p}.mlp.up_proj.weight"] = (I, H)
        out[f"{p}.mlp.down_proj.weight"] = (H, I)
    return out


def random_weights(cfg: Mapping, seed: int, *, dtype=torch.float32, scale: float = 0.02
                   ) -> Dict[str, torch.Tensor]:
    """Random tensors of the checkpoint's shapes: matrices N(0, scale), norm
    weights 1 + N(0, 0.01); rounded to ``dtype``."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in expected_tensor_shapes(cfg).items():
        x = torch.randn(shape, generator=g, dtype=torch.float32)
        if len(shape) == 1:
            x = 1.0 + 0.01 * x
        else:
            x = scale * x
        out[name] = x.to(dtype)
    return out
