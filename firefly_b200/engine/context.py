"""What one step looks like to the parts of a model: the batch's metadata on the
device, the caches, and scratch memory.

A step is a flat list of tokens from several requests.  Each token knows its
request (``token_seq``, an index into this step's sequences) and its absolute
position; that is all the kernels need to find its keys, whatever the cut.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Tuple

import torch


class Workspace:
    """Named scratch buffers, reused from layer to layer and from step to step.

    A buffer grows when a larger one is asked for, unless the workspace is
    frozen (while a CUDA graph that uses its addresses exists)."""

    def __init__(self, device):
        self.device = torch.device(device)
        self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        # the views handed out, by (tag, type, shape): a step asks for the same few hundred again and
        # again, and making a view costs the host several microseconds
        self._views: Dict[tuple, torch.Tensor] = {}
        self.frozen = False
        self.version = 0          # counts (re)allocations: graphs that captured an address note it

    def get(self, tag: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        vkey = (tag, dtype, tuple(shape))
        view = self._views.get(vkey)
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= int(s)
        key = (tag, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            if self.frozen:
                raise RuntimeError(f"workspace buffer '{tag}' would have to grow to {n} elements "
                                   "while a captured graph uses it")
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
            self.version += 1
            self._views.clear()   # views of the buffer that was replaced must not be handed out again
        if len(self._views) > 4096:
            self._views.clear()
        view = buf[:n].view(*shape)
        self._views[vkey] = view
        return view

    def get_zeroed(self, tag: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """A buffer that is zero when first handed out (and after it grows); users
        must leave it zero (counters that a kernel resets itself)."""
        key = (tag, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < numel:
            if self.frozen:
                raise RuntimeError(f"workspace buffer '{tag}' would have to grow while a captured graph uses it")
            buf = torch.zeros(max(numel, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
            self.version += 1
            self._views.clear()
        return buf[:numel]

    def zero(self, tag: str, dtype: torch.dtype) -> None:
        buf = self._bufs.get((tag, dtype))
        if buf is not None:
            buf.zero_()

    def reserve(self, tag: str, numel: int, dtype: torch.dtype) -> None:
        self.get(tag, (numel,), dtype)

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


@dataclass
class StepContext:
    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor            # int32 [T]
    positions: torch.Tensor            # int32 [T] absolute position of each token
    token_seq: torch.Tensor            # int32 [T] index of the token's sequence in this step
    cu_q: torch.Tensor                 # int32 [n+1] token offsets of the sequences
    ctx_lens: torch.Tensor             # int32 [n] tokens already in the cache
    state_slots: torch.Tensor          # int32 [n] fixed-size state slot of each sequence
    seq_fresh: torch.Tensor            # int32 [n] 1 when this is the request's first step
    logits_rows: torch.Tensor          # int32 [r] tokens whose logits are wanted
    block_tables: List[torch.Tensor]   # per KV group: int32 [n, max_blocks]
    q_lens: List[int]                  # host copies
    ctx_lens_host: List[int]
    max_q_len: int
    max_kv_len: int
    workspace: Workspace
    status: torch.Tensor               # int32 [1], set by a kernel that met a bad index
    cache: object                      # CacheManager
    dtype: torch.dtype                 # activation type of this engine
    pure_decode: bool = False
    num_decode_seqs: int = 0           # the first this-many sequences have exactly one token
    captured: bool = False             # being captured into a CUDA graph: launch shapes must be static
    ranges_by_length: bool = False     # the decoding sequences differ much in length (a hint for the attention)
    key_share_level: int = 0           # captured steps: over how many blocks at most a portion's keys may be shared out
    memo: Dict[tuple, object] = field(default_factory=dict)   # what layers work out alike for this step (slices, counts)

    def kv(self, slot: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Pages of cache slot ``slot`` and the block table of its group."""
        pages, g = self.cache.kv_view(slot)
        return pages, self.block_tables[g]

    def state(self, slot: int) -> torch.Tensor:
        """Fixed-size state tensor of cache slot ``slot``: [1+max_requests, *shape]."""
        return self.cache.state_storage[slot]
