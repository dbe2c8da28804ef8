"""The cache manager: paged keys/values in groups, block tables, state slots.

Cache slots (one per run of a layer that writes a cache) are grouped by what
they need: all slots with the same ``PagedKVSpec`` form a *group* that shares one
page pool, one allocator and, per request, one block table; a page id is valid in
every slot of its group.  Groups with a window give pages back as soon as the
window has passed them; all pages return when the request ends.  Beside the
pages, a request holds one *state slot*: an index into the fixed-size state
tensors that mixers with a ``StateSpec`` asked for (none for Qwen3 dense, which
leaves the slot empty).

The reference keeps one pool for all layers ([blocks,16,nkv,d] per layer,
src/engine.cc:105-113), one ``vector<int> block_table`` per request
(include/firefly/request.h:28) and never frees a finished request's pages except
through radix-tree eviction (src/scheduler.cc:165-186); prefix sharing is not
part of this engine, so pages go straight back to the free list.

This file is host logic only, except for ``allocate_storage`` which creates the
device tensors; the bookkeeping is usable (and tested) without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from .block_allocator import BlockAllocator, PageError
from .spec import PagedKVSpec, StateSpec

SCRATCH_PAGE = 0  # reserved in every group: padded lanes of a captured graph write here


class OutOfPages(RuntimeError):
    pass


@dataclass
class KVGroup:
    spec: PagedKVSpec
    slots: List[int]                      # cache slot ids, in order
    allocator: BlockAllocator
    storage: Optional[torch.Tensor] = None  # [n_slots, 1+num_blocks, 2, nkv, block, d]

    def slot_view(self, slot: int) -> torch.Tensor:
        return self.storage[self.slots.index(slot)]


@dataclass
class RequestCache:
    """What one live request holds."""

    request_id: object
    num_tokens: int = 0                   # tokens whose keys/values are in the cache
    tables: List[List[int]] = field(default_factory=list)   # per group; -1 = given back
    first_live: List[int] = field(default_factory=list)     # per group: first page index still held
    state_slot: int = -1
    fresh: bool = True                    # no step has run yet (state must start at zero)
    serial: int = 0                       # unique per admission (an id() may be reused, this is not)


class CacheManager:
    def __init__(self, slot_specs: Dict[int, object], *, block_size: int, num_blocks: int,
                 max_requests: int):
        """``slot_specs``: cache slot id -> PagedKVSpec | StateSpec | None.
        ``num_blocks``: usable pages per group (the scratch page comes on top)."""
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        self.block_size = block_size
        self.num_blocks = num_blocks
        self.max_requests = max_requests
        self.groups: List[KVGroup] = []
        self.slot_group: Dict[int, int] = {}
        self.state_specs: Dict[int, StateSpec] = {}
        self.state_storage: Dict[int, torch.Tensor] = {}
        by_spec: Dict[PagedKVSpec, int] = {}
        for slot in sorted(slot_specs):
            spec = slot_specs[slot]
            if spec is None:
                continue
            if isinstance(spec, PagedKVSpec):
                if spec not in by_spec:
                    by_spec[spec] = len(self.groups)
                    self.groups.append(KVGroup(spec, [], BlockAllocator(num_blocks, first_id=1)))
                g = by_spec[spec]
                self.groups[g].slots.append(slot)
                self.slot_group[slot] = g
            elif isinstance(spec, StateSpec):
                self.state_specs[slot] = spec
            else:
                raise TypeError(f"cache slot {slot}: unknown cache spec {spec!r}")
        # state slots: index 0 is scratch (padded lanes), requests get 1..max_requests
        self._free_state = list(range(max_requests, 0, -1))
        self.live: Dict[object, RequestCache] = {}
        self._serial = 0

    # ---- sizes ----------------------------------------------------------------
    def bytes_per_block(self, dtype: torch.dtype) -> int:
        es = torch.empty((), dtype=dtype).element_size()
        return sum(len(g.slots) * 2 * g.spec.num_kv_heads * self.block_size * g.spec.head_dim * es
                   for g in self.groups)

    def allocate_storage(self, dtype: torch.dtype, device) -> None:
        for g in self.groups:
            g.storage = torch.zeros((len(g.slots), 1 + self.num_blocks, 2, g.spec.num_kv_heads,
                                     self.block_size, g.spec.head_dim), dtype=dtype, device=device)
        for slot, spec in self.state_specs.items():
            self.state_storage[slot] = torch.zeros((1 + self.max_requests, *spec.shape),
                                                   dtype=spec.dtype, device=device)

    def kv_view(self, slot: int) -> Tuple[torch.Tensor, int]:
        """(pages of this slot [1+num_blocks, 2, nkv, block, d], group index)."""
        g = self.slot_group[slot]
        return self.groups[g].slot_view(slot), g

    # ---- requests -------------------------------------------------------------
    def admit(self, request_id) -> RequestCache:
        if request_id in self.live:
            raise PageError(f"request {request_id!r} is already live")
        if not self._free_state:
            raise OutOfPages(f"no free request slot (max_requests={self.max_requests})")
        self._serial += 1
        rc = RequestCache(request_id, 0, [[] for _ in self.groups], [0 for _ in self.groups],
                          self._free_state.pop(), True, self._serial)
        self.live[request_id] = rc
        return rc

    def can_admit(self) -> bool:
        return bool(self._free_state)

    def _first_needed_page(self, g: KVGroup, ctx: int) -> int:
        """Index of the first page that a query at position >= ctx can still read."""
        if g.spec.window is None:
            return 0
        return max(0, ctx - g.spec.window + 1) // self.block_size

    def pages_needed(self, rc: RequestCache, new_total: int) -> List[int]:
        need = -(-new_total // self.block_size)
        return [max(0, need - len(t)) for t in rc.tables]

    def can_grow(self, rc: RequestCache, new_total: int, reserve: int = 0) -> bool:
        return all(g.allocator.num_free - reserve >= n
                   for g, n in zip(self.groups, self.pages_needed(rc, new_total)))

    def grow(self, rc: RequestCache, new_total: int) -> bool:
        """Make room for ``new_total`` tokens in every group; all or nothing."""
        needs = self.pages_needed(rc, new_total)
        if not all(g.allocator.can_allocate(n) for g, n in zip(self.groups, needs)):
            return False
        for g, n, table in zip(self.groups, needs, rc.tables):
            got = g.allocator.allocate(n)
            assert got is not None
            table.extend(got)
        return True

    def advance(self, rc: RequestCache, n_tokens: int) -> None:
        """``n_tokens`` more tokens are now in the cache; give back pages that a
        window has passed."""
        rc.num_tokens += n_tokens
        rc.fresh = False
        if rc.tables and rc.num_tokens > min(len(t) for t in rc.tables) * self.block_size:
            raise PageError(f"request {rc.request_id!r} holds {rc.num_tokens} tokens in "
                            f"{[len(t) for t in rc.tables]} pages of {self.block_size}")
        for gi, g in enumerate(self.groups):
            first = self._first_needed_page(g, rc.num_tokens)
            table = rc.tables[gi]
            if first > rc.first_live[gi]:
                passed = [b for b in table[rc.first_live[gi]:first] if b >= 0]
                g.allocator.free(passed)
                for i in range(rc.first_live[gi], first):
                    table[i] = -1
                rc.first_live[gi] = first

    def free(self, rc: RequestCache) -> None:
        if self.live.get(rc.request_id) is not rc:
            raise PageError(f"request {rc.request_id!r} is not live (freed twice?)")
        for g, table in zip(self.groups, rc.tables):
            g.allocator.free([b for b in table if b >= 0])
            table.clear()
        self._free_state.append(rc.state_slot)
        rc.state_slot = -1
        rc.num_tokens = 0
        del self.live[rc.request_id]

    # ---- invariants (tests) -----------------------------------------------------
    def check(self) -> None:
        for gi, g in enumerate(self.groups):
            g.allocator.check()
            held = []
            for rc in self.live.values():
                held.extend(b for b in rc.tables[gi] if b >= 0)
            if len(held) != len(set(held)):
                raise PageError(f"group {gi}: a page is held by two requests")
            if len(held) != g.allocator.num_held:
                raise PageError(f"group {gi}: {g.allocator.num_held} pages are out, requests hold "
                                f"{len(held)}")
        slots = [rc.state_slot for rc in self.live.values()]
        if len(slots) != len(set(slots)) or len(slots) + len(self._free_state) != self.max_requests:
            raise PageError("state slots lost or held twice")

    @property
    def num_free_blocks(self) -> int:
        return min((g.allocator.num_free for g in self.groups), default=self.num_blocks)
