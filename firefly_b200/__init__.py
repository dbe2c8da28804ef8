"""firefly_b200: a small, whole LLM inference engine for one NVIDIA B200.

Everything between a request's tokens and its next token for Qwen3 dense, built
from parts that another architecture can reuse: typed configuration and an
architecture registry, safetensors weights bound by name, layers assembled from
mixer / feed-forward / norm / position parts, a paged cache with per-request
block tables, one step function for mixed batches, a scheduler, samplers and
hand-written sm_100a kernels.
"""
from . import models as _models  # noqa: F401  (registers the architectures)

__version__ = "0.1.0"
