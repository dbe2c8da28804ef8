"""The weight arena on the device: each tensor once, fused in place, the same bits from a folder
and from the seed, any stored type, any file offset."""
import json
import os
import struct

import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu


def _cfg(raw):
    from firefly_b200.models import config_from_dict
    return config_from_dict(raw)


def _bound_tensors(model):
    out = []
    for b in model.blocks:
        out += [b.mixer.w_qkv, b.mixer.w_o, b.mixer.q_norm_w, b.mixer.k_norm_w, b.feed_forward.w_gate_up,
                b.feed_forward.w_down, *(n.weight for n in b.norms)]
    out += [model.embedding.table, model.final_norm.weight, model.head.weight]
    return out


@pytest.mark.parametrize("raw,dtype", [(P.TINY_A, "bfloat16"), (P.TINY_B, "bfloat16"), (P.TINY_B, "float32"),
                                       (P.TINY_C, "bfloat16")])
def test_seed_and_folder_give_the_same_arena_bit_for_bit(tmp_path, raw, dtype):
    from firefly_b200.engine.loading import load_model, random_model
    from firefly_b200.weights import write_random_model
    cfg = _cfg(raw)
    tdt = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    d = write_random_model(cfg, 11, str(tmp_path / "m"), dtype=tdt)          # drawn on the CPU
    from_file, _ = load_model(d, dtype=dtype)
    from_seed = random_model(cfg, 11, dtype=dtype)                            # drawn by the kernel
    a, b = from_file.weight_arena, from_seed.weight_arena
    assert a.plan.slots == b.plan.slots
    for name in a.plan.slots:
        assert torch.equal(a.view(name), b.view(name)), name
    other = random_model(cfg, 12, dtype=dtype)
    assert not torch.equal(other.weight_arena.view("model.embed_tokens.weight"), a.view("model.embed_tokens.weight"))


@pytest.mark.parametrize("raw", [P.TINY_A, P.TINY_C])
def test_arena_is_the_only_copy_of_the_weights(tmp_path, raw):
    from firefly_b200.engine.loading import load_model
    from firefly_b200.weights import write_random_model
    d = write_random_model(_cfg(raw), 3, str(tmp_path / "m"), dtype=torch.bfloat16)
    load_model(d, dtype="bfloat16")                   # first load: builds the module, makes library handles
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    before = torch.cuda.memory_allocated()
    model, _ = load_model(d, dtype="bfloat16")
    torch.cuda.synchronize()
    arena = model.weight_arena
    lo, hi = arena.buffer.data_ptr(), arena.buffer.data_ptr() + arena.buffer.numel()
    for t in _bound_tensors(model):
        assert lo <= t.data_ptr() and t.data_ptr() + t.numel() * t.element_size() <= hi
    # nothing but the arena (and the rotary table, shared between the layers) was allocated
    extra = torch.cuda.memory_allocated() - before - arena.buffer.numel()
    assert 0 <= extra <= 1 << 20, extra
    assert model.load_facts["arena_bytes"] == arena.plan.total_bytes and model.load_facts["files"] == 1
    assert model.load_facts["pinned_files"] in (0, 1)


def test_fused_tensors_are_the_sources_in_their_rows(tmp_path):
    from firefly_b200.engine.loading import load_model
    from firefly_b200.ops.kernels import interleave_gate_up
    from firefly_b200.weights import write_random_model
    raw = P.TINY_D                                                     # intermediate 272 = 17 groups of 16
    d = write_random_model(_cfg(raw), 4, str(tmp_path / "m"), dtype=torch.bfloat16)
    model, _ = load_model(d, dtype="bfloat16")
    from firefly_b200.weights import SafetensorsFile
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    src = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    for i, b in enumerate(model.blocks):
        p = f"model.layers.{i}"
        qkv = torch.cat([src[f"{p}.self_attn.{x}_proj.weight"] for x in "qkv"], dim=0)
        assert torch.equal(b.mixer.w_qkv.cpu(), qkv)
        gu = interleave_gate_up(src[f"{p}.mlp.gate_proj.weight"], src[f"{p}.mlp.up_proj.weight"])
        assert b.feed_forward.interleaved and torch.equal(b.feed_forward.w_gate_up.cpu(), gu)
    # a 32-bit engine stacks gate and up (no interleave) and widens exactly
    model32, _ = load_model(d, dtype="float32")
    b = model32.blocks[0]
    want = torch.cat([src["model.layers.0.mlp.gate_proj.weight"], src["model.layers.0.mlp.up_proj.weight"]]).float()
    assert not b.feed_forward.interleaved and torch.equal(b.feed_forward.w_gate_up.cpu(), want)


def _write_with_odd_header(path, tensors):
    """A safetensors file whose data does not start on an even address."""
    header, blobs, off = {}, [], 0
    names = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.float64: "F64"}
    for n, t in tensors.items():
        raw = t.contiguous().view(torch.uint8).numpy().tobytes()
        header[n] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    blob = json.dumps(header).encode()
    if len(blob) % 2 == 0:
        blob += b" "
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for b in blobs:
            fh.write(b)


@pytest.mark.parametrize("stored", [torch.float32, torch.float16, torch.float64, torch.bfloat16])
@pytest.mark.parametrize("weight_dtype", ["keep", "engine"])
def test_any_stored_type_and_any_file_offset(tmp_path, stored, weight_dtype, monkeypatch):
    from firefly_b200.engine.loading import load_model
    from firefly_b200.weights import arena as A
    monkeypatch.setattr(A, "STAGING_BYTES", 4096)         # conversions then run in several pieces
    raw = P.TINY_D
    w = {k: v.to(stored) for k, v in P.random_weights(raw, 9, scale=0.05).items()}
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(raw))
    _write_with_odd_header(str(d / "model.safetensors"), w)
    model, _ = load_model(str(d), dtype="bfloat16", weight_dtype=weight_dtype)
    wide = stored in (torch.float32, torch.float64) and weight_dtype == "keep"
    want_dt = torch.float32 if wide else torch.bfloat16
    for i, b in enumerate(model.blocks):
        p = f"model.layers.{i}"
        o = b.mixer.w_o
        assert o.dtype == want_dt and torch.equal(o.cpu(), w[f"{p}.self_attn.o_proj.weight"].to(want_dt))
        qkv = torch.cat([w[f"{p}.self_attn.{x}_proj.weight"].to(want_dt) for x in "qkv"], dim=0)
        assert torch.equal(b.mixer.w_qkv.cpu(), qkv)
        g, u = (w[f"{p}.mlp.{x}_proj.weight"].to(want_dt) for x in ("gate", "up"))
        from firefly_b200.ops.kernels import interleave_gate_up
        want = interleave_gate_up(g, u) if want_dt == torch.bfloat16 else torch.cat([g, u])
        assert torch.equal(b.feed_forward.w_gate_up.cpu(), want)
        assert b.norms[0].weight.dtype == torch.float32
        assert torch.equal(b.norms[0].weight.cpu(), w[f"{p}.input_layernorm.weight"].to(torch.float32))
