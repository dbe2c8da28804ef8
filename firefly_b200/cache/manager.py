"""The cache manager: paged keys/values in groups, block tables, state slots.

Cache slots (one per run of a layer that writes a cache) are grouped by what
they need: all slots with the same ``PagedKVSpec`` form a *group* that shares one
page pool, one allocator and, per request, one block table; a page id is valid in
every slot of its group.  Every group has its own page size and its own number of
pages: a group whose layers only ever read a window of keys needs far fewer pages
than one that keeps every key, and a mixer may ask for a page size of its own.
Groups with a window give pages back as soon as the window has passed them; all
pages return when the request ends.  Beside the
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
from typing import Dict, List, Optional, Sequence, Tuple, Union

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
    block_size: int                       # tokens per page of this group
    num_blocks: int                       # usable pages of this group (the scratch page comes on top)
    allocator: BlockAllocator
    storage: Optional[torch.Tensor] = None  # [n_slots, 1+num_blocks, 2, nkv, block, d]

    def bytes_per_token(self, dtype: torch.dtype) -> int:
        es = torch.empty((), dtype=dtype).element_size()
        return len(self.slots) * 2 * self.spec.num_kv_heads * self.spec.head_dim * es

    def pages_for(self, ctx: int, new_tokens: int) -> int:
        """Pages a request must hold in this group to run ``new_tokens`` tokens behind ``ctx`` cached
        ones (counting from the first page a window still needs)."""
        last = -(-(ctx + new_tokens) // self.block_size)
        first = 0 if self.spec.window is None else max(0, ctx - self.spec.window + 1) // self.block_size
        return last - first

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


def plan_groups(slot_specs: Dict[int, object], block_size: int) -> List[Tuple[PagedKVSpec, List[int], int]]:
    """Which groups the cache slots form: (spec, slot ids, page size) in a fixed order.  The engine
    sizes each group from this before it makes the manager."""
    order: List[PagedKVSpec] = []
    slots: Dict[PagedKVSpec, List[int]] = {}
    for slot in sorted(slot_specs):
        spec = slot_specs[slot]
        if isinstance(spec, PagedKVSpec):
            if spec not in slots:
                slots[spec] = []
                order.append(spec)
            slots[spec].append(slot)
    return [(sp, slots[sp], int(sp.block_size or block_size)) for sp in order]


class CacheManager:
    def __init__(self, slot_specs: Dict[int, object], *, block_size: int,
                 num_blocks: Union[int, Sequence[int]], max_requests: int):
        """``slot_specs``: cache slot id -> PagedKVSpec | StateSpec | None.  ``block_size``: tokens per
        page for groups that ask for none of their own.  ``num_blocks``: usable pages (the scratch
        page comes on top), one number for every group or one per group in ``plan_groups`` order."""
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        self.block_size = block_size
        self.max_requests = max_requests
        self.groups: List[KVGroup] = []
        self.slot_group: Dict[int, int] = {}
        self.state_specs: Dict[int, StateSpec] = {}
        self.state_storage: Dict[int, torch.Tensor] = {}
        planned = plan_groups(slot_specs, block_size)
        counts = [int(num_blocks)] * len(planned) if isinstance(num_blocks, int) else [int(n) for n in num_blocks]
        if len(counts) != len(planned):
            raise ValueError(f"{len(counts)} page counts for {len(planned)} cache groups")
        for (spec, slots, bs), n in zip(planned, counts):
            if bs <= 0 or n < 0:
                raise ValueError("page size must be positive and page count non-negative")
            for slot in slots:
                self.slot_group[slot] = len(self.groups)
            self.groups.append(KVGroup(spec, list(slots), bs, n, BlockAllocator(n, first_id=1)))
        for slot in sorted(slot_specs):
            spec = slot_specs[slot]
            if spec is None or isinstance(spec, PagedKVSpec):
                continue
            if isinstance(spec, StateSpec):
                self.state_specs[slot] = spec
            else:
                raise TypeError(f"cache slot {slot}: unknown cache spec {spec!r}")
        # state slots: index 0 is scratch (padded lanes), requests get 1..max_requests
        self._free_state = list(range(max_requests, 0, -1))
        self.live: Dict[object, RequestCache] = {}
        self._serial = 0

    @property
    def num_blocks(self) -> int:
        """Pages of the smallest group (all groups are equal when one number was given)."""
        return min((g.num_blocks for g in self.groups), default=0)

    # ---- sizes ----------------------------------------------------------------
    def bytes_per_block(self, dtype: torch.dtype) -> int:
        """Bytes of one page of every group together (equal page sizes: bytes per ``block_size`` tokens)."""
        return sum(g.bytes_per_token(dtype) * g.block_size for g in self.groups)

    def allocate_storage(self, dtype: torch.dtype, device) -> None:
        for g in self.groups:
            g.storage = torch.zeros((len(g.slots), 1 + g.num_blocks, 2, g.spec.num_kv_heads,
                                     g.block_size, g.spec.head_dim), dtype=dtype, device=device)
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
        return max(0, ctx - g.spec.window + 1) // g.block_size

    def pages_needed(self, rc: RequestCache, new_total: int) -> List[int]:
        """New pages per group for the request to hold ``new_total`` tokens (a table keeps the places of
        pages that were given back, so its length counts every page the request ever had)."""
        return [max(0, -(-new_total // g.block_size) - len(t)) for g, t in zip(self.groups, rc.tables)]

    def why_it_cannot_fit(self, total_tokens: int, portion: int) -> Optional[str]:
        """None if a request of ``total_tokens`` tokens, fed at most ``portion`` at a time, could run with
        the pools to itself; else which group is too small."""
        for gi, g in enumerate(self.groups):
            if g.spec.window is None:
                need = -(-total_tokens // g.block_size)
            else:
                need = -(-(min(total_tokens, g.spec.window + portion)) // g.block_size) + 1
                need = min(need, -(-total_tokens // g.block_size))
            if need > g.num_blocks:
                return (f"its {total_tokens} tokens need {need} pages of {g.block_size} in cache group {gi}, "
                        f"which has {g.num_blocks}")
        return None

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
        if any(rc.num_tokens > len(t) * g.block_size for g, t in zip(self.groups, rc.tables)):
            raise PageError(f"request {rc.request_id!r} holds {rc.num_tokens} tokens in "
                            f"{[len(t) for t in rc.tables]} pages of {[g.block_size for g in self.groups]}")
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
        return min((g.allocator.num_free for g in self.groups), default=0)
