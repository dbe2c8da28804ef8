"""A generation request as the scheduler sees it.

Fields follow the reference's ``GenerationRequest`` (include/firefly/request.h:11-41):
id, prompt_tokens, generated_tokens, max_tokens, status PENDING / ACTIVE /
FINISHED, the block table and context length (held here by ``cache``).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import List, Optional

from ..cache.manager import RequestCache
from ..sampling.params import SamplingParams


class RequestStatus(enum.Enum):
    PENDING = "pending"
    ACTIVE = "active"
    FINISHED = "finished"


@dataclass
class GenerationRequest:
    id: str
    prompt_tokens: List[int]
    sampling: SamplingParams = field(default_factory=SamplingParams)
    generated_tokens: List[int] = field(default_factory=list)
    status: RequestStatus = RequestStatus.PENDING
    cache: Optional[RequestCache] = None
    finish_reason: Optional[str] = None      # "eos" | "length" | "error: ..."
    num_preemptions: int = 0
    arrival: int = 0

    @property
    def max_tokens(self) -> int:
        return self.sampling.max_tokens

    def get_total_len(self) -> int:
        return len(self.prompt_tokens) + len(self.generated_tokens)

    @property
    def context_len(self) -> int:
        """Tokens whose keys and values are in the cache."""
        return self.cache.num_tokens if self.cache is not None else 0

    def token_at(self, i: int) -> int:
        n = len(self.prompt_tokens)
        return self.prompt_tokens[i] if i < n else self.generated_tokens[i - n]

    def tokens_between(self, lo: int, hi: int) -> List[int]:
        n = len(self.prompt_tokens)
        if hi <= n:
            return self.prompt_tokens[lo:hi]
        if lo >= n:
            return self.generated_tokens[lo - n:hi - n]
        return self.prompt_tokens[lo:] + self.generated_tokens[:hi - n]
