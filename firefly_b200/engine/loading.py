"""From a model folder (or a configuration and a seed) to a bound model."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..config.base import ModelConfig
from ..models.decoder import DecoderModel
from ..models.registry import load_config, spec_for
from ..ops import kernels as K
from ..parts import Runtime
from ..weights.arena import RandomSource, WeightArena
from ..weights.loader import load_weights, plan_arena

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(d) -> torch.dtype:
    if isinstance(d, torch.dtype):
        if d not in (torch.bfloat16, torch.float32):
            raise ValueError(f"engine dtype must be bfloat16 or float32, got {d}")
        return d
    try:
        return _DTYPES[str(d).lower()]
    except KeyError:
        raise ValueError(f"engine dtype must be bfloat16 or float32, got {d!r}") from None


def require_cuda(device) -> torch.device:
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError("firefly_b200 runs on a CUDA device only (there is no CPU path)")
    if not torch.cuda.is_available():
        raise RuntimeError("firefly_b200 needs a CUDA device and none is available")
    return dev


def load_config_with_file_hints(model_dir: str) -> ModelConfig:
    """The typed configuration of a model folder.  A config.json that says nothing about
    ``tie_word_embeddings`` is read as tied when the weight file holds no ``lm_head.weight``
    (checkpoints with a shared head usually store the matrix once)."""
    from ..config.base import read_config_json
    from ..models.registry import config_from_dict
    from ..weights.safetensors_io import open_model_files
    raw = read_config_json(model_dir)
    if "tie_word_embeddings" not in raw:
        files = open_model_files(model_dir)
        try:
            names = {n for f in files for n in f.entries}
        finally:
            for f in files:
                f.close()
        if "lm_head.weight" not in names and "model.embed_tokens.weight" in names:
            raw = dict(raw, tie_word_embeddings=True)
    return config_from_dict(raw)


def load_model(model_dir: str, *, dtype="bfloat16", device="cuda:0", weight_dtype: str = "keep"
               ) -> Tuple[DecoderModel, ModelConfig]:
    """Read ``config.json``, pick the model by its architecture name, bind the tensors of
    ``model.safetensors`` by name.  The weights lie in one device arena (``model.weight_arena``);
    ``model.load_facts`` tells its size and whether the file could be pinned.  ``weight_dtype``:
    "keep" leaves tensors stored in 32-bit as they are, "engine" narrows them to the engine's type."""
    dt = parse_dtype(dtype)
    config = load_config_with_file_hints(model_dir)          # a folder's faults are told before the machine's
    dev = require_cuda(device)
    K.set_exact_matmul()
    model = DecoderModel(spec_for(config), Runtime(dev, dt))
    tensors, arena, facts = load_weights(model_dir, model, dtype=dt, device=dev, weight_dtype=weight_dtype)
    model.bind(tensors)
    model.weight_arena, model.load_facts = arena, facts
    return model, config


def random_model(config: ModelConfig, seed: int, *, dtype="bfloat16", device="cuda:0",
                 num_layers: Optional[int] = None) -> DecoderModel:
    """A model of ``config``'s shape with seeded random weights drawn on the device (no folder is
    written): the same values, bit for bit, that ``write_random_model`` stores for this seed."""
    dt = parse_dtype(dtype)
    dev = require_cuda(device)
    K.set_exact_matmul()
    model = DecoderModel(spec_for(config), Runtime(dev, dt))
    specs = [w for w in model.weight_specs() if not w.optional]
    stored = torch.bfloat16 if dt == torch.bfloat16 else torch.float32
    available = {w.name: (tuple(w.shape), stored if w.kind == "float" else torch.int32) for w in specs}
    plan, names = plan_arena(model, available, dtype=dt)
    arena = WeightArena(plan, dev)
    RandomSource(specs, seed, stored).fill(arena, names)
    model.bind(arena.tensors())
    model.weight_arena, model.load_facts = arena, {"arena_bytes": plan.total_bytes}
    return model
