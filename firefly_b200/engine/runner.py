"""The step function: a batch of (request, its next tokens) through the model.

``ModelRunner.step(entries)`` runs exactly the tokens it is given, as one batch,
against the cache that earlier steps left, and returns 32-bit logits at the
wanted places.  Portions of prompts and single decoded tokens may sit side by
side, cut anywhere.  The reference instead runs each prefill portion as a call
of its own and all decodes as another (src/engine.cc:238-342) through a
rectangular ``forward(input_ids[B,S], context_lens[B], ...)``
(include/firefly/model/model.h:45-46).

Per step the host packs all integer metadata (token ids, positions, the token ->
sequence map, block tables, wanted rows) into one pinned buffer and uploads it
with one copy.  The block tables of a step are as wide as the longest table among
its requests, not as wide as the model's longest context, so the copy grows with
the pages that are live (the reference uploads a table as wide as the whole pool
every step, src/engine.cc:96,126,321).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, OutOfPages, RequestCache
from ..models.decoder import DecoderModel
from ..ops import kernels as K
from .context import StepContext, Workspace


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places among them
    (indices into ``tokens``) whose logits are wanted."""

    cache: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepError(RuntimeError):
    pass


_STATUS = {1: "a token id outside the vocabulary reached the embedding kernel",
           2: "a token's cache page is missing from its block table (write)",
           3: "a position beyond the rotary table",
           4: "a key's cache page is missing from a block table (read)",
           101: "matrix product: the loader's wait for a free stage ran out",
           102: "matrix product: the wait for a loaded stage ran out",
           103: "matrix product: the wait for the accumulator ran out",
           107: "attention (tcgen05): a bounded wait ran out"}


def status_text(code: int) -> str:
    return _STATUS.get(int(code), "unknown")


class StatusRead:
    """The device status word on its way to the host: queued behind a step's work, readable
    without a stall once the host has waited for anything queued after it."""

    __slots__ = ("buf", "event")

    def __init__(self, buf: torch.Tensor, event: "torch.cuda.Event"):
        self.buf, self.event = buf, event

    def code(self) -> int:
        self.event.synchronize()
        return int(self.buf[0])


class MetaLayout:
    """Where each integer array of a step lies in the packed metadata buffer."""

    def __init__(self, T: int, n: int, r: int, widths: Sequence[int], update_cap: int = 0):
        """``widths``: entries per row of each cache group's block table.  ``update_cap`` > 0 reserves
        room for that many (index, value) pairs in front of the tables: changes to tables that stay
        on the device (see ``DecodeGraphs``)."""
        self.T, self.n, self.r, self.widths = T, n, r, [int(w) for w in widths]
        self.update_cap = update_cap
        off = 0

        def take(count):
            nonlocal off
            lo = off
            off += (count + 3) // 4 * 4     # keep every array 16-byte aligned
            return lo
        self.token_ids = take(T)
        self.positions = take(T)
        self.token_seq = take(T)
        self.cu_q = take(n + 1)
        self.ctx_lens = take(n)
        self.state_slots = take(n)
        self.seq_fresh = take(n)
        self.logits_rows = take(r)
        self.updates = take(1 + 2 * update_cap) if update_cap else off
        self.head_size = off                   # everything in front of the block tables
        self.tables = [take(n * w) for w in self.widths]
        self.size = off


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, *, max_model_len: int,
                 max_batched_tokens: int = 8192, max_seqs: int = 256):
        self.model = model
        self.cache = cache
        self.device = model.rt.device
        self.dtype = model.rt.dtype
        self.vocab_size = model.spec.vocab_size
        self.max_model_len = max_model_len
        # widest block table a request can have, per cache group (each group has its own page size)
        self.max_blocks = [-(-max_model_len // g.block_size) for g in cache.groups]
        self.workspace = Workspace(self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._meta_cap = 0
        self._meta_ring: List[list] = []      # [pinned buffer, event of its last upload]
        self._meta_turn = 0
        self._meta_dev: Optional[torch.Tensor] = None
        self._ensure_meta(MetaLayout(max_batched_tokens, max_seqs, max_seqs, self.max_blocks).size)
        self._status_ring = [[torch.zeros(1, dtype=torch.int32).pin_memory(), None] for _ in range(self.META_RING)]
        self._status_turn = 0
        self.steps_run = 0
        self.kernel_launches = 0

    def queue_status_read(self) -> StatusRead:
        """Queue a copy of the status word to pinned memory behind the work that is on the stream
        now.  The engine looks at it when it reads the step's tokens, so a kernel that met a bad
        index or gave up a wait is noticed at the step it happened in, without an extra stall."""
        slot = self._status_ring[self._status_turn]
        self._status_turn = (self._status_turn + 1) % len(self._status_ring)
        if slot[1] is not None:
            slot[1].synchronize()
        else:
            slot[1] = torch.cuda.Event()
        slot[0].copy_(self.status, non_blocking=True)
        slot[1].record()
        return StatusRead(slot[0], slot[1])

    def clear_status(self) -> None:
        self.status.zero_()

    # ------------------------------------------------------------------------------
    META_RING = 4     # pinned metadata buffers in rotation

    def _ensure_meta(self, size: int) -> None:
        if size > self._meta_cap:
            self._meta_cap = size
            self._meta_ring = [[torch.empty(size, dtype=torch.int32).pin_memory(), None]
                               for _ in range(self.META_RING)]
            self._meta_turn = 0
            self._meta_dev = torch.empty(size, dtype=torch.int32, device=self.device)

    def _next_meta_host(self) -> list:
        """The pinned buffer for the next step's metadata.  The upload of a step is only queued
        when ``step`` returns, and a step without wanted logits is never waited for, so the host
        may be several steps ahead of the device: a buffer is written again only after the upload
        that last read it has happened."""
        slot = self._meta_ring[self._meta_turn]
        self._meta_turn = (self._meta_turn + 1) % self.META_RING
        if slot[1] is not None:
            slot[1].synchronize()
        return slot

    def build_context(self, entries: Sequence[StepEntry], *, meta_host: Optional[torch.Tensor] = None,
                      meta_dev: Optional[torch.Tensor] = None, upload: bool = True) -> StepContext:
        # sequences that decode one token come first in the step's arrays (in their given order), the
        # others after them: the attention kernels for the two kinds then each see one contiguous range
        n = len(entries)
        given = list(entries)
        order = sorted(range(n), key=lambda i: 0 if len(given[i].tokens) == 1 else 1)
        entries = [given[i] for i in order]
        q_lens = [len(e.tokens) for e in entries]
        T = sum(q_lens)
        ctx_lens = [e.cache.num_tokens for e in entries]
        starts = {}
        pos = 0
        for e, ql in zip(entries, q_lens):
            starts[id(e)] = pos
            pos += ql
        wants: List[int] = []          # in the order the caller gave the entries
        for e in given:
            ql = len(e.tokens)
            for w in e.want:
                if not (0 <= w < ql):
                    raise StepError(f"request {e.cache.request_id!r}: wanted place {w} is outside its "
                                    f"{ql} tokens of this step")
                wants.append(starts[id(e)] + w)
        # tables as wide as this step's longest (in steps of four entries), not as the longest possible
        widths = [min(cap, max(4, -(-max(len(e.cache.tables[g]) for e in entries) // 4) * 4))
                  for g, cap in enumerate(self.max_blocks)]
        lay = MetaLayout(T, n, len(wants), widths)
        slot = None
        if meta_host is None:
            self._ensure_meta(lay.size)
            slot = self._next_meta_host()
            meta_host, meta_dev = slot[0], self._meta_dev
        elif lay.size > meta_host.numel():
            raise StepError("metadata buffer too small for this step")
        h = meta_host.numpy()
        pos = 0
        for i, (e, ql, cl) in enumerate(zip(entries, q_lens, ctx_lens)):
            toks = np.asarray(e.tokens, dtype=np.int64)
            if toks.size and (toks.min() < 0 or toks.max() >= self.vocab_size):
                raise StepError(f"request {e.cache.request_id!r}: token id outside [0, {self.vocab_size})")
            if cl + ql > self.max_model_len:
                raise StepError(f"request {e.cache.request_id!r}: {cl + ql} tokens exceed the engine's "
                                f"max_model_len {self.max_model_len}")
            h[lay.token_ids + pos: lay.token_ids + pos + ql] = toks
            h[lay.positions + pos: lay.positions + pos + ql] = np.arange(cl, cl + ql)
            h[lay.token_seq + pos: lay.token_seq + pos + ql] = i
            h[lay.cu_q + i] = pos
            h[lay.ctx_lens + i] = cl
            h[lay.state_slots + i] = e.cache.state_slot
            h[lay.seq_fresh + i] = 1 if e.cache.fresh else 0
            for g, table in enumerate(e.cache.tables):
                need_pages = -(-(cl + ql) // self.cache.groups[g].block_size)
                if len(table) < need_pages:
                    raise OutOfPages(f"request {e.cache.request_id!r} has {len(table)} pages in group "
                                     f"{g}, this step needs {need_pages}")
                w = lay.widths[g]
                row = lay.tables[g] + i * w
                h[row: row + len(table)] = table
                h[row + len(table): row + w] = -1
            pos += ql
        h[lay.cu_q + n] = pos
        if wants:
            h[lay.logits_rows: lay.logits_rows + len(wants)] = wants
        if upload:
            meta_dev[:lay.size].copy_(meta_host[:lay.size], non_blocking=True)
            if slot is not None:
                if slot[1] is None:
                    slot[1] = torch.cuda.Event()
                slot[1].record()
        return self.context_from_layout(lay, meta_dev, q_lens, ctx_lens)

    def context_from_layout(self, lay: MetaLayout, meta_dev: torch.Tensor, q_lens: List[int],
                            ctx_lens: List[int]) -> StepContext:
        d = meta_dev

        def sl(off, count):
            return d[off: off + count]
        return StepContext(
            num_tokens=lay.T, num_seqs=lay.n,
            token_ids=sl(lay.token_ids, lay.T), positions=sl(lay.positions, lay.T),
            token_seq=sl(lay.token_seq, lay.T), cu_q=sl(lay.cu_q, lay.n + 1),
            ctx_lens=sl(lay.ctx_lens, lay.n), state_slots=sl(lay.state_slots, lay.n),
            seq_fresh=sl(lay.seq_fresh, lay.n), logits_rows=sl(lay.logits_rows, lay.r),
            block_tables=[sl(o, lay.n * w).view(lay.n, w) for o, w in zip(lay.tables, lay.widths)],
            q_lens=list(q_lens), ctx_lens_host=list(ctx_lens),
            max_q_len=max(q_lens, default=0),
            max_kv_len=max((c + q for c, q in zip(ctx_lens, q_lens)), default=0),
            workspace=self.workspace, status=self.status, cache=self.cache, dtype=self.dtype,
            pure_decode=all(q == 1 for q in q_lens), num_decode_seqs=sum(1 for q in q_lens if q == 1),
            ranges_by_length=K.lengths_differ_much([c for c, q in zip(ctx_lens, q_lens) if q == 1]))

    # ------------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the entries' tokens as one batch.  Returns float32 logits
        [number of wanted places, vocab] in the order of the entries and of each
        entry's ``want`` (a view of scratch memory: valid until the next step).
        Every entry's request must already hold the pages for its new tokens."""
        entries = [e for e in entries if len(e.tokens)]
        if not entries:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        ids = [id(e.cache) for e in entries]
        if len(set(ids)) != len(ids):
            raise StepError("a request appears twice in one step")
        ctx = self.build_context(entries)
        logits = self.model.forward(ctx)
        for e in entries:
            self.cache.advance(e.cache, len(e.tokens))
        self.steps_run += 1
        return logits

    def check_status(self) -> None:
        """Raise if a kernel met a bad index since the last check (synchronises)."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise StepError(f"device status {code}: {_STATUS.get(code, 'unknown')}")
