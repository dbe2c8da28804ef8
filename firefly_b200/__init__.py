"""firefly_b200: a small, whole LLM inference engine for one NVIDIA B200.

Everything between a request's tokens and its next token for Qwen3 dense, built
from parts that another architecture can reuse: typed configuration and an
architecture registry, safetensors weights bound by name, layers assembled from
mixer / feed-forward / norm / position parts, a paged cache with per-request
block tables, one step function for mixed batches, a scheduler, samplers and
hand-written sm_100a kernels.

    from firefly_b200 import LLM
    out = LLM("model_dir", dtype="bfloat16").generate([[1, 2, 3]], max_tokens=8)
"""
from . import models as _models  # noqa: F401  (registers the architectures)
from .sampling.params import SamplingParams

__version__ = "0.1.0"


def __getattr__(name):
    # the engine imports torch.cuda machinery; load it on first use
    if name in ("LLM", "Engine", "EngineOptions", "ResultQueue", "StepOutput"):
        from . import entry
        return getattr(entry, name)
    raise AttributeError(name)


__all__ = ["LLM", "Engine", "EngineOptions", "ResultQueue", "StepOutput", "SamplingParams"]
