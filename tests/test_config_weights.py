"""Configuration, registry and weight loading (no GPU)."""
import json
import os
import struct

import pytest
import torch

import plain_qwen3 as P
from firefly_b200.config import ConfigError, Qwen3Config, ScheduleEntry
from firefly_b200.models import (config_from_dict, expected_weights, known_architectures, load_config,
                                 spec_for)
from firefly_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, read_weights,
                                  save_safetensors, write_random_model)
from firefly_b200.weights.loader import storage_dtype


def test_config_reads_every_key():
    cfg = config_from_dict(P.TINY_B)
    assert isinstance(cfg, Qwen3Config)
    for k in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
              "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings", "rms_norm_eps",
              "rope_theta", "tie_word_embeddings"):
        assert getattr(cfg, k) == P.TINY_B[k]
    assert cfg.to_dict()["architectures"] == ["Qwen3ForCausalLM"]


def test_config_defaults_follow_reference():
    raw = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128,
               num_hidden_layers=1, num_attention_heads=4, vocab_size=100)
    cfg = config_from_dict(raw)
    assert cfg.num_key_value_heads == 4 and cfg.head_dim == 16
    assert cfg.max_position_embeddings == 32768 and cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 10000.0
    assert cfg.tie_word_embeddings is False


@pytest.mark.parametrize("patch,msg", [
    ({"hidden_size": None}, "hidden_size"),
    ({"num_attention_heads": 5, "num_key_value_heads": 2}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"attention_bias": True}, "attention_bias"),
    ({"use_sliding_window": True}, "sliding"),
    ({"layer_types": ["full_attention", "sliding_attention"]}, "layer_types"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"num_hidden_layers": "3"}, "integer"),
])
def test_config_rejects(patch, msg):
    raw = dict(P.TINY_A)
    raw.update(patch)
    with pytest.raises(ConfigError, match=msg):
        config_from_dict(raw)


def test_unknown_architecture_lists_known():
    raw = dict(P.TINY_A, architectures=["NoSuchModel"])
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        config_from_dict(raw)
    assert "Qwen3ForCausalLM" in known_architectures()


def test_spec_is_data():
    spec = spec_for(config_from_dict(P.TINY_B))
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert spec.layers[0].mixer.params["num_kv_heads"] == 2
    assert spec.layers[0].position.params["theta"] == 1e6
    assert spec.resolved_schedule() == [(0, 0, True), (1, 1, True), (2, 2, True)]
    import dataclasses
    bad = dataclasses.replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1, cache=5, write_cache=False)))
    with pytest.raises(ConfigError, match="no earlier run writes"):
        bad.resolved_schedule()
    twice = dataclasses.replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(0), ScheduleEntry(1, cache=0, write_cache=False)))
    assert twice.resolved_schedule() == [(0, 0, True), (0, 1, True), (1, 0, False)]


def test_expected_weights_match_checkpoint_names():
    for raw in (P.TINY_A, P.TINY_B, P.TINY_C):
        ws = expected_weights(spec_for(config_from_dict(raw)))
        got = {w.name: w.shape for w in ws if not w.optional}
        assert got == P.expected_tensor_shapes(raw)


def test_safetensors_roundtrip_and_foreign_writer(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
         "c": torch.arange(6, dtype=torch.int64).view(2, 3), "d": torch.randn(2, 2).to(torch.float16)}
    p1 = str(tmp_path / "own.safetensors")
    save_safetensors(p1, t)
    from safetensors.torch import load_file, save_file
    back = load_file(p1)                       # our writer, their reader
    for k in t:
        assert torch.equal(back[k], t[k])
    p2 = str(tmp_path / "theirs.safetensors")
    save_file(t, p2)                           # their writer, our reader
    f = SafetensorsFile(p2)
    for k in t:
        assert torch.equal(f.tensor(k), t[k]) and f.tensor(k).dtype == t[k].dtype
    with pytest.raises(SafetensorsError, match="not found"):
        f.tensor("zzz")
    f.close()


def test_safetensors_corrupt_files(tmp_path):
    p = tmp_path / "x.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(SafetensorsError, match="too small"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header size"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)      # truncated data
    with pytest.raises(SafetensorsError, match="outside the file"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [5], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)     # shape x dtype != bytes
    with pytest.raises(SafetensorsError, match="needs 20"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(str(p))


def _folder(tmp_path, raw, weights, name="m"):
    d = tmp_path / name
    d.mkdir()
    (d / "config.json").write_text(json.dumps(raw))
    save_safetensors(str(d / "model.safetensors"), weights)
    return str(d)


def test_load_weights_reports_everything_at_once(tmp_path):
    raw = P.TINY_B
    w = P.random_weights(raw, 0)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(10, 10)
    w["extra.tensor"] = torch.zeros(3)
    w["model.layers.2.input_layernorm.weight"] = torch.zeros(96, dtype=torch.int32)
    d = _folder(tmp_path, raw, w)
    spec = spec_for(load_config(d))
    with pytest.raises(WeightError) as ei:
        read_weights(d, expected_weights(spec), dtype=torch.float32)
    e = ei.value
    assert set(e.missing) == {"model.layers.1.mlp.up_proj.weight", "model.norm.weight"}
    assert e.unexpected == ["extra.tensor"]
    assert e.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (10, 10), (192, 96))]
    assert e.wrong_kind == [("model.layers.2.input_layernorm.weight", "int", "float")]
    for frag in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "extra.tensor",
                 "file has [10, 10], model needs [192, 96]"):
        assert frag in str(e)


def test_load_weights_dtype_policy(tmp_path):
    raw = P.TINY_A
    w = P.random_weights(raw, 0)
    w = {k: (v.to(torch.bfloat16) if "mlp" in k else v) for k, v in w.items()}
    w["lm_head.weight"] = torch.zeros(256, 64)          # a tied head stored anyway is ignored
    d = _folder(tmp_path, raw, w)
    spec = spec_for(load_config(d))
    got = read_weights(d, expected_weights(spec), dtype=torch.bfloat16)
    assert got["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16      # kept in bfloat16
    assert got["model.layers.0.self_attn.q_proj.weight"].dtype == torch.float32  # stored 32-bit stays
    assert torch.equal(got["model.layers.0.self_attn.q_proj.weight"], w["model.layers.0.self_attn.q_proj.weight"])
    got32 = read_weights(d, expected_weights(spec), dtype=torch.float32)
    assert all(t.dtype == torch.float32 for t in got32.values())
    assert storage_dtype(torch.int64, torch.bfloat16) == torch.int32
    assert storage_dtype(torch.uint8, torch.float32) == torch.int32
    assert storage_dtype(torch.float16, torch.bfloat16) == torch.bfloat16


def test_tied_head_is_inferred_when_the_key_is_absent(tmp_path):
    from firefly_b200.engine.loading import load_config_with_file_hints
    raw = {k: v for k, v in P.TINY_A.items() if k != "tie_word_embeddings"}
    w = P.random_weights(P.TINY_A, 0)                      # no lm_head.weight
    d = _folder(tmp_path, raw, w, "tied")
    assert load_config_with_file_hints(d).tie_word_embeddings is True
    w["lm_head.weight"] = torch.zeros(256, 64)
    d2 = _folder(tmp_path, raw, w, "untied")
    assert load_config_with_file_hints(d2).tie_word_embeddings is False
    d3 = _folder(tmp_path, dict(raw, tie_word_embeddings=False), P.random_weights(P.TINY_A, 0), "says_untied")
    assert load_config_with_file_hints(d3).tie_word_embeddings is False      # what config.json says stands


def test_missing_files(tmp_path):
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(P.TINY_A))
    spec = spec_for(load_config(str(tmp_path)))
    with pytest.raises(SafetensorsError, match="model.safetensors"):
        read_weights(str(tmp_path), expected_weights(spec), dtype=torch.float32)


def test_random_model_folder(tmp_path):
    cfg = config_from_dict(P.TINY_B)
    d = write_random_model(cfg, 7, str(tmp_path / "r"), dtype=torch.bfloat16)
    assert load_config(d) == cfg
    spec = spec_for(cfg)
    a = read_weights(d, expected_weights(spec), dtype=torch.bfloat16)
    d2 = write_random_model(cfg, 7, str(tmp_path / "r2"), dtype=torch.bfloat16)
    b = read_weights(d2, expected_weights(spec), dtype=torch.bfloat16)
    d3 = write_random_model(cfg, 8, str(tmp_path / "r3"), dtype=torch.bfloat16)
    c = read_weights(d3, expected_weights(spec), dtype=torch.bfloat16)
    assert all(torch.equal(a[k], b[k]) for k in a)                 # same seed, same weights
    assert not torch.equal(a["lm_head.weight"], c["lm_head.weight"])
    # matrices stay bfloat16; norm weights are read in 32-bit arithmetic and are widened once, on the way in
    assert all(v.dtype == (torch.float32 if v.dim() == 1 else torch.bfloat16) for v in a.values())
    q = a["model.layers.0.self_attn.q_proj.weight"].float()
    n = a["model.norm.weight"].float()
    assert abs(q.std().item() - 0.02) < 0.002 and abs(n.mean().item() - 1.0) < 0.01
    # a sharded folder loads the same
    os.remove(os.path.join(d, "model.safetensors"))
    names = sorted(a)
    half = len(names) // 2
    save_safetensors(os.path.join(d, "s1.safetensors"), {k: a[k].to(torch.bfloat16) for k in names[:half]})
    save_safetensors(os.path.join(d, "s2.safetensors"), {k: a[k].to(torch.bfloat16) for k in names[half:]})
    wm = {k: ("s1.safetensors" if i < half else "s2.safetensors") for i, k in enumerate(names)}
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": wm}, fh)
    s = read_weights(d, expected_weights(spec), dtype=torch.bfloat16)
    assert all(torch.equal(a[k], s[k]) for k in a)
