from . import qwen3  # noqa: F401  (registers Qwen3ForCausalLM)
from .decoder import DecoderModel, expected_weights
from .registry import (architecture_of, config_from_dict, known_architectures, load_config,
                       register_architecture, spec_for)

__all__ = ["DecoderModel", "expected_weights", "architecture_of", "config_from_dict",
           "known_architectures", "load_config", "register_architecture", "spec_for"]
