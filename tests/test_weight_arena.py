"""The weight arena's plan, the counter-based random weights and the file mapping (no GPU needed)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from firefly_b200.models import config_from_dict, expected_weights, spec_for
from firefly_b200.models.decoder import DecoderModel
from firefly_b200.parts import Runtime
from firefly_b200.weights import (ArenaPlan, FusedSpec, MappedFile, Piece, SafetensorsError, WeightSpec, draw_cpu,
                                  plan_arena, read_weights, save_safetensors)
from firefly_b200.weights import random_init as R
from firefly_b200.weights.arena import ALIGN


def _model(raw, dtype=torch.bfloat16):
    return DecoderModel(spec_for(config_from_dict(raw)), Runtime(torch.device("cpu"), dtype))


@pytest.mark.parametrize("raw", [P.TINY_A, P.TINY_B, P.TINY_C])
def test_plan_holds_every_tensor_once_and_fuses(raw):
    model = _model(raw)
    avail = {w.name: (tuple(w.shape), torch.bfloat16) for w in model.weight_specs() if not w.optional}
    plan, names = plan_arena(model, avail, dtype=torch.bfloat16)
    plan.check()
    assert set(names) == set(avail)
    L = raw["num_hidden_layers"]
    # the sources of fused tensors have no slot of their own; everything else has exactly one
    for i in range(L):
        p = f"model.layers.{i}"
        for leaf in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "mlp.gate_proj", "mlp.up_proj"):
            assert f"{p}.{leaf}.weight" not in plan.slots
        assert plan.slots[f"{p}.self_attn.qkv_proj.weight"].shape == (
            (raw["num_attention_heads"] + 2 * raw["num_key_value_heads"]) * raw["head_dim"], raw["hidden_size"])
        assert plan.slots[f"{p}.mlp.gate_up_proj.weight"].shape == (2 * raw["intermediate_size"], raw["hidden_size"])
        assert plan.slots[f"{p}.input_layernorm.weight"].dtype == torch.float32      # read in 32-bit arithmetic
    payload = sum(int(np.prod(s)) * (4 if len(s) == 1 else 2) for s, _ in avail.values())
    assert payload <= plan.total_bytes <= payload + ALIGN * len(plan.slots)
    # gate and up interleave in groups of 16 rows when the width allows, else they are stacked
    pl = plan.placements["model.layers.0.mlp.up_proj.weight"]
    if raw["intermediate_size"] % 16 == 0:
        assert (pl.row0, pl.group, pl.group_stride) == (16, 16, 32)
    else:
        assert pl.row0 == raw["intermediate_size"] and pl.group == raw["intermediate_size"]


def test_plan_mixed_sources_take_the_wider_type_and_errors():
    srcs = {"a": ((4, 8), torch.bfloat16), "b": ((4, 8), torch.float32), "c": ((3,), torch.float32)}
    plan = ArenaPlan(srcs, [FusedSpec("ab", (8, 8), (Piece("a", 0), Piece("b", 4)))])
    assert plan.slots["ab"].dtype == torch.float32 and set(plan.slots) == {"ab", "c"}
    with pytest.raises(ValueError, match="does not fit"):
        ArenaPlan(srcs, [FusedSpec("ac", (8, 8), (Piece("a", 0), Piece("c", 4)))])
    with pytest.raises(KeyError, match="not loaded"):
        ArenaPlan(srcs, [FusedSpec("ax", (8, 8), (Piece("a", 0), Piece("x", 4)))])
    with pytest.raises(ValueError, match="no multiple"):
        ArenaPlan(srcs, [FusedSpec("ab", (8, 8), (Piece("a", 0, 3, 6), Piece("b", 4)))])


def test_random_values_are_a_function_of_seed_name_and_index():
    w = WeightSpec("model.layers.0.mlp.up_proj.weight", (48, 40))
    a = draw_cpu(w, 5, dtype=torch.float32)
    assert torch.equal(a, draw_cpu(w, 5, dtype=torch.float32))
    assert not torch.equal(a, draw_cpu(w, 6, dtype=torch.float32))
    assert not torch.equal(a, draw_cpu(WeightSpec("other", (48, 40)), 5, dtype=torch.float32))
    # a taller tensor of the same name starts with the same values: the index alone decides
    tall = draw_cpu(WeightSpec(w.name, (96, 40)), 5, dtype=torch.float32)
    assert torch.equal(tall[:48], a)
    # bfloat16 storage is the 32-bit draw rounded once
    assert torch.equal(draw_cpu(w, 5, dtype=torch.bfloat16), a.to(torch.bfloat16))
    ints = draw_cpu(WeightSpec("table", (1000,), kind="int", init="int:7"), 1, dtype=torch.float32)
    assert ints.dtype == torch.int32 and int(ints.min()) == 0 and int(ints.max()) == 6


def test_random_laws():
    big = draw_cpu(WeightSpec("m", (512, 512)), 0, dtype=torch.float32).double()
    assert abs(big.mean().item()) < 2e-4 and abs(big.std().item() - 0.02) < 2e-4
    # the shape of the law, not only its first two moments: kurtosis and tail mass of a normal
    z = big / 0.02
    assert abs((z ** 4).mean().item() - 3.0) < 0.05
    assert abs((z.abs() > 2).double().mean().item() - 0.0455) < 0.003
    nrm = draw_cpu(WeightSpec("n", (4096,), init="norm"), 0, dtype=torch.float32).double()
    assert abs(nrm.mean().item() - 1.0) < 1e-3 and abs(nrm.std().item() - 0.01) < 1e-3
    assert torch.equal(draw_cpu(WeightSpec("z", (5,), init="zeros"), 0, dtype=torch.float32), torch.zeros(5))
    assert torch.equal(draw_cpu(WeightSpec("o", (5,), init="ones"), 0, dtype=torch.bfloat16),
                       torch.ones(5, dtype=torch.bfloat16))
    t = R.normal_table()
    assert t.dtype == torch.int32 and t.numel() == 65537 and int(t[32768]) == 0
    assert torch.equal(t, -t.flip(0)) and bool((t[1:] >= t[:-1]).all())


def test_mapping_without_registration_and_with_a_refused_one(tmp_path):
    path = str(tmp_path / "blob.bin")
    data = bytes(range(256)) * 40
    with open(path, "wb") as fh:
        fh.write(data)
    for register in (False, True):
        # on a machine without a GPU the registration is refused by the driver: not an error, the
        # file stays pageable
        m = MappedFile(path, register=register)
        assert m.size == len(data) and m.address != 0
        if not torch.cuda.is_available():
            assert m.pinned is False
        got = (np.ctypeslib.as_array((np.ctypeslib.ctypes.c_ubyte * m.size).from_address(m.address))).tobytes()
        assert got == data
        m.close()
        m.close()                                                    # closing twice is harmless
    with pytest.raises(OSError, match="cannot map"):
        MappedFile(str(tmp_path / "absent.bin"))


def test_truncated_file_is_refused_before_anything_is_copied(tmp_path):
    raw = P.TINY_A
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(raw))
    save_safetensors(str(d / "model.safetensors"), P.random_weights(raw, 0))
    full = (d / "model.safetensors").read_bytes()
    (d / "model.safetensors").write_bytes(full[: len(full) - 100])
    with pytest.raises(SafetensorsError, match="outside the file"):
        read_weights(str(d), expected_weights(spec_for(config_from_dict(raw))), dtype=torch.float32)
    (hlen,) = struct.unpack("<Q", full[:8])
    (d / "model.safetensors").write_bytes(full[: 8 + hlen // 2])
    with pytest.raises(SafetensorsError, match="invalid header size"):
        read_weights(str(d), expected_weights(spec_for(config_from_dict(raw))), dtype=torch.float32)


def test_weight_dtype_option(tmp_path):
    raw = P.TINY_A
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(raw))
    w = P.random_weights(raw, 0)                                     # stored in 32-bit
    save_safetensors(str(d / "model.safetensors"), w)
    exp = expected_weights(spec_for(config_from_dict(raw)))
    keep = read_weights(str(d), exp, dtype=torch.bfloat16)
    narrow = read_weights(str(d), exp, dtype=torch.bfloat16, weight_dtype="engine")
    name = "model.layers.0.self_attn.o_proj.weight"
    assert keep[name].dtype == torch.float32 and narrow[name].dtype == torch.bfloat16
    assert torch.equal(narrow[name], w[name].to(torch.bfloat16))
    assert narrow["model.norm.weight"].dtype == torch.float32
    with pytest.raises(ValueError, match="weight_dtype"):
        read_weights(str(d), exp, dtype=torch.bfloat16, weight_dtype="fp8")
