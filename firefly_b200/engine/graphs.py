"""Decode steps replayed from CUDA graphs.

A step in which every request decodes one token has the same launches whatever
the requests are; only the integer metadata differs.  For each batch-size bucket
(the reference's {1,2,4,8,16,32,64}, include/firefly/engine.h:72, captured in
src/engine.cc:121-169) the model's forward and the arg-max are captured once
over a static metadata buffer; a decode step then fills that buffer, uploads it
with one copy and replays.  The captured sampler reads a temperature, a seed and a
counter per lane from a second static buffer, so requests that sample with a
temperature run from the same graph as greedy ones (a lane with temperature 0 is an
arg-max) and their tokens, too, can feed the next step without leaving the device.
Unused lanes of a bucket decode a dummy token at
position 0 into the reserved scratch page, so they never touch a live page.
Unlike the reference, the block-table rows are bounded by the model length, not
by the size of the whole pool, and nothing is allocated inside the capture.

The block tables of a bucket stay on the device.  A step uploads only the head of
the metadata (tokens, positions, lengths: a few hundred bytes) and a short list
of (index, value) pairs, the table entries that changed since the last replay (a
lane's new page, a new request's row); a small kernel at the front of the graph
writes them into the tables.  When more entries changed than the list holds (a
bucket's first use, many new requests at once) the whole buffer is uploaded that
once.  So the bytes a decode step moves do not grow with the model's longest
context (the reference copies a table as wide as the whole pool every step,
src/engine.cc:96,126,321).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from collections import OrderedDict

from ..cache.manager import SCRATCH_PAGE, OutOfPages
from ..ops import kernels as K
from .context import Workspace
from .runner import MetaLayout, ModelRunner, StepEntry, StepError


class _Bucket:
    __slots__ = ("size", "layout", "meta_host", "meta_stage", "meta_dev", "graph", "logits", "tokens", "h_tokens",
                 "events", "launches", "lanes", "turn", "by_length", "samp_stage", "samp_dev", "samp_greedy", "h_status",
                 "changes", "full_upload", "q_lens", "rows", "starts", "stage_events")


class LaunchedStep:
    """A replay that has been put on the stream: its tokens arrive in ``h_tokens`` once
    ``event`` has passed."""
    __slots__ = ("bucket", "n", "h_tokens", "event", "logits", "h_status", "status_code")


class _Capture:
    """``torch.cuda.graph`` with the one failure a model of foreign parts can cause turned into words:
    an operation that synchronises with the host (``.item()``, an index taken from a device tensor,
    ``bool(t.any())``) ends the capture with an error."""

    def __init__(self, graph):
        self._cm = torch.cuda.graph(graph)

    def __enter__(self):
        return self._cm.__enter__()

    def __exit__(self, et, ev, tb):
        try:
            self._cm.__exit__(et, ev, tb)
        except RuntimeError as e:
            raise StepError("the model's step could not be captured into a CUDA graph: some part read a device "
                            "value on the host. Declare host_synchronous = True on that part (parts/base.py) "
                            f"or run with use_cuda_graphs=False. ({str(e).splitlines()[0]})") from e
        if et is not None and issubclass(et, RuntimeError) and "capture" in str(ev):
            raise StepError("the model's step could not be captured into a CUDA graph: some part read a device "
                            "value on the host. Declare host_synchronous = True on that part (parts/base.py) "
                            f"or run with use_cuda_graphs=False. ({str(ev).splitlines()[0]})") from ev
        return False


class DecodeGraphs:
    def __init__(self, runner: ModelRunner, batch_sizes: Sequence[int]):
        self.runner = runner
        self.sizes = sorted(set(int(b) for b in batch_sizes))
        self.workspace = Workspace(runner.device)
        self.buckets: Dict[int, _Bucket] = {}
        self.replays = 0
        self.replays_by_length = 0
        self.kernel_launches = 0
        self.h2d_bytes = 0            # metadata bytes uploaded by all replays so far
        self.full_uploads = 0
        # steps of other shapes (prompt portions, alone or beside decode tokens) whose shape came again
        self.shapes: "OrderedDict[tuple, _Bucket]" = OrderedDict()
        self.shape_seen: Dict[tuple, int] = {}
        self.shape_workspace = Workspace(runner.device)
        self.shape_replays = 0
        self.shape_captures = 0

    def supports(self, n: int) -> bool:
        return bool(self.sizes) and n <= self.sizes[-1]

    def _bucket_for(self, n: int) -> _Bucket:
        size = next(b for b in self.sizes if b >= n)
        if size not in self.buckets:
            if not self.workspace.frozen:
                # one eager run at the largest size gives every scratch buffer its final
                # extent, so no captured address ever moves
                self._prepare(self.sizes[-1], capture=False)
                self.workspace.frozen = True
            self.buckets[size] = self._prepare(size, capture=True)
        return self.buckets[size]

    def _fill(self, b: _Bucket, entries: Sequence[StepEntry]) -> None:
        """Write the step's metadata into the bucket's pinned buffer.  A lane that holds the same
        request as in the step before only gets what changed: its token, position and any new
        page.  Every write into a block table is also noted in ``b.changes`` (offset, values), from
        which the step's update list is made."""
        r, lay = self.runner, b.layout
        h = b.meta_host.numpy()
        n = len(entries)
        if b.lanes is None:
            # constant parts, and every lane as padding: a dummy token at position 0 in the scratch page
            h[lay.token_ids: lay.token_ids + b.size] = 0
            h[lay.positions: lay.positions + b.size] = 0
            h[lay.token_seq: lay.token_seq + b.size] = np.arange(b.size)
            h[lay.cu_q: lay.cu_q + b.size + 1] = np.arange(b.size + 1)
            h[lay.ctx_lens: lay.ctx_lens + b.size] = 0
            h[lay.state_slots: lay.state_slots + b.size] = 0
            h[lay.seq_fresh: lay.seq_fresh + b.size] = 0
            h[lay.logits_rows: lay.logits_rows + b.size] = np.arange(b.size)
            for off, w in zip(lay.tables, lay.widths):
                tab = h[off: off + b.size * w].reshape(b.size, w)
                tab[:, 0] = SCRATCH_PAGE
                tab[:, 1:] = -1
            b.lanes = [None] * b.size
            b.full_upload = True

        def put(off, values):
            h[off: off + len(values)] = values
            b.changes.append((off, values))
        for i in range(n, b.size):                 # lanes that fell out of use become padding again
            if b.lanes[i] is not None:
                h[lay.token_ids + i] = 0
                h[lay.positions + i] = 0
                h[lay.ctx_lens + i] = 0
                h[lay.state_slots + i] = 0
                h[lay.seq_fresh + i] = 0
                for off, w in zip(lay.tables, lay.widths):
                    put(off + i * w, [SCRATCH_PAGE])        # position 0 reads and writes the first entry only
                b.lanes[i] = None
        for i, e in enumerate(entries):
            rc = e.cache
            cl = rc.num_tokens
            tok = int(e.tokens[0])
            if not (0 <= tok < r.vocab_size):
                raise ValueError(f"token id {tok} outside the vocabulary")
            if cl + 1 > r.max_model_len:
                raise ValueError(f"request {rc.request_id!r} exceeds max_model_len")
            h[lay.token_ids + i] = tok
            h[lay.positions + i] = cl
            h[lay.ctx_lens + i] = cl
            h[lay.seq_fresh + i] = 1 if rc.fresh else 0
            old = b.lanes[i]
            same = old is not None and old[0] == rc.serial
            if not same:
                h[lay.state_slots + i] = rc.state_slot
            lens = []
            for g, table in enumerate(rc.tables):
                row = lay.tables[g] + i * lay.widths[g]
                if same and old[2][g] == rc.first_live[g] and old[1][g] <= len(table):
                    if old[1][g] < len(table):
                        put(row + old[1][g], table[old[1][g]:])
                else:
                    # entries behind the request's pages are never read (a key's page index is below its
                    # count of pages), so what an earlier request left there may stay
                    put(row, list(table))
                lens.append(len(table))
            b.lanes[i] = (rc.serial, lens, list(rc.first_live))

    def _write_updates(self, b: _Bucket) -> bool:
        """The step's table changes as (index, value) pairs in the buffer's update list.  False if
        they do not fit: then the whole buffer has to be uploaded."""
        lay = b.layout
        h = b.meta_host.numpy()
        count = sum(len(v) for _, v in b.changes)
        fits = count <= lay.update_cap and not b.full_upload
        if fits:
            k = lay.updates + 1
            for off, values in b.changes:
                m = len(values)
                h[k: k + 2 * m: 2] = np.arange(off, off + m)
                h[k + 1: k + 1 + 2 * m: 2] = values
                k += 2 * m
        h[lay.updates] = count if fits else 0
        b.changes = []
        b.full_upload = False
        return fits

    def _prepare(self, size: int, capture: bool) -> _Bucket:
        r = self.runner
        b = _Bucket()
        b.size = size
        b.layout = MetaLayout(size, size, size, r.max_blocks, update_cap=max(64, 4 * size))
        b.changes, b.full_upload = [], True
        b.meta_host = torch.zeros(b.layout.size, dtype=torch.int32).pin_memory()
        # two of everything the host touches while a replay may still be using the other
        b.meta_stage = [torch.zeros(b.layout.size, dtype=torch.int32).pin_memory() for _ in range(2)]
        b.meta_dev = torch.zeros(b.layout.size, dtype=torch.int32, device=r.device)
        b.tokens = torch.zeros(size, dtype=torch.int32, device=r.device)
        # per lane: seed (int64), counter (int64), temperature (float32), in this order so that the
        # 64-bit values are aligned whatever the size; all zero = every lane greedy
        b.samp_stage = [torch.zeros(5 * size, dtype=torch.int32).pin_memory() for _ in range(2)]
        b.samp_dev = torch.zeros(5 * size, dtype=torch.int32, device=r.device)
        b.samp_greedy = True
        b.h_tokens = [torch.zeros(size, dtype=torch.int32).pin_memory() for _ in range(2)]
        b.h_status = [torch.zeros(1, dtype=torch.int32).pin_memory() for _ in range(2)]
        b.events = [torch.cuda.Event() for _ in range(2)]
        b.turn = 0
        b.lanes = None
        self._fill(b, [])
        self._write_updates(b)
        b.full_upload = True                  # the first replay uploads everything once more
        b.meta_dev.copy_(b.meta_host)
        ctx = r.context_from_layout(b.layout, b.meta_dev, [1] * size, [0] * size)
        ctx.workspace = self.workspace
        ctx.max_kv_len = r.max_model_len      # launch shapes must not depend on the requests
        ctx.captured = True
        ctx.num_decode_seqs = size
        side = torch.cuda.Stream(device=r.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._apply_updates(b)
            logits = r.model.forward(ctx)     # warm-up: library handles, lazy module loads
            self._sample(b, logits)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(r.device)
        if not capture:
            return b
        b.graph = torch.cuda.CUDAGraph()
        before = K.LAUNCHES
        with _Capture(b.graph):
            self._apply_updates(b)
            b.logits = r.model.forward(ctx)
            self._sample(b, b.logits)
        b.launches = K.LAUNCHES - before      # own kernels in one replay
        # A second graph of the same step for requests of very different lengths, if any kernel
        # makes something of that hint (the attention then shares its blocks out by length).
        # Both graphs work on the same buffers; (graph, logits, launches) or None.
        b.by_length = None
        ctx.ranges_by_length = True
        calls = K.BY_LENGTH_CALLS
        with torch.cuda.stream(side):
            r.model.forward(ctx)              # warm-up of the kernels that only this form uses
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(r.device)
        if K.BY_LENGTH_CALLS != calls:
            g2 = torch.cuda.CUDAGraph()
            before = K.LAUNCHES
            with _Capture(g2):
                self._apply_updates(b)
                logits2 = r.model.forward(ctx)
                self._sample(b, logits2)
            b.by_length = (g2, logits2, K.LAUNCHES - before)
        return b

    def _apply_updates(self, b: _Bucket) -> None:
        """First kernel of a replay: the uploaded (index, value) pairs go into the block tables."""
        lay = b.layout
        if lay.tables:
            K.scatter_int(b.meta_dev, b.meta_dev[lay.updates:], lay.update_cap)

    def _sample(self, b: _Bucket, logits: torch.Tensor) -> None:
        d, n = b.samp_dev, b.size
        K.sample(logits, b.tokens, d[4 * n:].view(torch.float32), d[:2 * n].view(torch.int64),
                 d[2 * n: 4 * n].view(torch.int64))

    def _upload_sampling(self, b: _Bucket, k: int, sampling) -> None:
        """Per-lane (temperature, seed, counter) for the next replay; nothing is copied while
        every lane stays greedy."""
        greedy = sampling is None or all(t <= 0 for t, _, _ in sampling)
        if greedy and b.samp_greedy:
            return
        stage = b.samp_stage[k]
        h, n = stage.numpy(), b.size
        h[:] = 0
        if not greedy:
            m = len(sampling)
            h[:2 * n].view(np.int64)[:m] = [seed for _, seed, _ in sampling]
            h[2 * n: 4 * n].view(np.int64)[:m] = [counter for _, _, counter in sampling]
            h[4 * n:].view(np.float32)[:m] = [max(t, 0.0) for t, _, _ in sampling]
        b.samp_dev.copy_(stage, non_blocking=True)
        b.samp_greedy = greedy

    def launch(self, entries: Sequence[StepEntry], want_tokens: bool = True,
               tokens_from_last_replay: bool = False, sampling=None) -> LaunchedStep:
        """Put one decode step for ``entries`` (one token each) on the stream without waiting
        for it.  With ``tokens_from_last_replay`` the token of lane i is taken, on the device,
        from what this bucket's previous replay sampled for lane i (the host does not know it
        yet; the ids in ``entries`` are placeholders).  At most two launched steps of a bucket may
        be outstanding.  ``sampling``: per entry (temperature, seed, tokens generated so far),
        or None when every request is greedy."""
        n = len(entries)
        b = self._bucket_for(n)
        self._fill(b, entries)
        k = b.turn
        b.turn ^= 1
        self._upload_sampling(b, k, sampling)
        stage = b.meta_stage[k]
        # the head (tokens, positions, lengths, the update list) always; the tables only when more of
        # them changed than the list holds
        upto = b.layout.head_size if self._write_updates(b) else b.layout.size
        self.full_uploads += upto == b.layout.size
        stage[:upto].copy_(b.meta_host[:upto])
        b.meta_dev[:upto].copy_(stage[:upto], non_blocking=True)
        self.h2d_bytes += 4 * upto
        if tokens_from_last_replay:
            lay = b.layout
            b.meta_dev[lay.token_ids: lay.token_ids + n].copy_(b.tokens[:n], non_blocking=True)
        graph, logits, launches = b.graph, b.logits, b.launches
        if b.by_length is not None and K.lengths_differ_much([e.cache.num_tokens for e in entries]):
            graph, logits, launches = b.by_length
            self.replays_by_length += 1
        graph.replay()
        self.replays += 1
        self.kernel_launches += launches
        step = LaunchedStep()
        step.bucket, step.n, step.logits = b, n, logits[:n]
        step.h_tokens, step.event, step.h_status, step.status_code = None, None, None, 0
        if want_tokens:
            step.h_tokens = b.h_tokens[k]
            step.h_tokens[:n].copy_(b.tokens[:n], non_blocking=True)
            step.h_status = b.h_status[k]              # the status word rides behind the tokens
            step.h_status.copy_(self.runner.status, non_blocking=True)
            step.event = b.events[k]
            step.event.record()
        for e in entries:
            self.runner.cache.advance(e.cache, 1)
        self.runner.steps_run += 1
        return step

    # ------------------------------------------------------------------------------------------
    # Steps of any shape.  The launches of a step depend on its shape alone: how many tokens each
    # sequence brings (one-token sequences first) and which rows' logits are wanted.  While a long
    # prompt comes in in portions, or a set of requests decodes beside it, that shape repeats step
    # after step; queueing its ~330 launches from the host costs about as long as the device needs for
    # a 256-token step of the 8B shape and many times longer for small models.  So a shape that comes a
    # second time is captured (over metadata of its own, like a decode bucket: the head is uploaded
    # every step, block-table entries through the update list) and replayed from then on.
    MAX_SHAPES = 24            # captured shapes kept (the least recently used one goes)
    SHAPE_MAX_TOKENS = 1024    # longer steps are bound by the device, not by the host
    CAPTURE_AT = 2             # a shape is captured when it is seen this many times

    @staticmethod
    def shape_of(entries: Sequence[StepEntry]):
        """(order, key): the entries' order in the step (one-token sequences first, as the step function
        sorts them) and the shape key: tokens per sequence, wanted rows among the step's tokens, and how
        long the longest portion's context is in four coarse levels (a captured step fixes over how many
        blocks a portion's keys are shared out, and what suits 500 keys does not suit 16 000)."""
        order = sorted(range(len(entries)), key=lambda i: 0 if len(entries[i].tokens) == 1 else 1)
        q_lens = tuple(len(entries[i].tokens) for i in order)
        start, starts = 0, {}
        for i, ql in zip(order, q_lens):
            starts[i] = start
            start += ql
        rows = tuple(starts[i] + w for i, e in enumerate(entries) for w in e.want)
        key_tiles = max((-(-(e.cache.num_tokens + len(e.tokens)) // 64) for e in entries if len(e.tokens) > 1), default=0)
        level = 0 if key_tiles < 8 else (2 if key_tiles < 16 else (4 if key_tiles < 32 else 8))
        return order, (q_lens, rows, level)

    def shape_ready(self, entries: Sequence[StepEntry]):
        """The plan of a step that should run from a graph: (order, key), or None if its shape has not
        come often enough yet (it is counted), is too long, or the entries are not fit for it."""
        if not entries or len(entries) > self.runner.cache.max_requests:
            return None
        order, key = self.shape_of(entries)
        q_lens, rows, _ = key
        if sum(q_lens) > self.SHAPE_MAX_TOKENS or any(ql < 1 for ql in q_lens):
            return None
        if key not in self.shapes:
            seen = self.shape_seen.get(key, 0) + 1
            if len(self.shape_seen) > 4096:
                self.shape_seen.clear()
            self.shape_seen[key] = seen
            if seen < self.CAPTURE_AT:
                return None
        return order, key

    def _prepare_shape(self, key) -> _Bucket:
        """Capture one forward (and the sampler) for steps of shape ``key``, over metadata in which every
        sequence lies in the scratch page and the scratch state slot: the capture and the run before it
        write no live page and no request's state."""
        r = self.runner
        q_lens, rows, level = key
        n, T, nr = len(q_lens), sum(q_lens), len(rows)
        b = _Bucket()
        b.size, b.q_lens, b.rows = n, list(q_lens), list(rows)
        b.layout = lay = MetaLayout(T, n, max(nr, 1), r.max_blocks, update_cap=max(64, 4 * n))
        b.changes, b.full_upload = [], True
        b.meta_host = torch.zeros(lay.size, dtype=torch.int32).pin_memory()
        b.meta_stage = [torch.zeros(lay.size, dtype=torch.int32).pin_memory() for _ in range(2)]
        b.stage_events = [None, None]
        b.meta_dev = torch.zeros(lay.size, dtype=torch.int32, device=r.device)
        b.tokens = torch.zeros(max(nr, 1), dtype=torch.int32, device=r.device)
        b.samp_stage = [torch.zeros(5 * max(nr, 1), dtype=torch.int32).pin_memory() for _ in range(2)]
        b.samp_dev = torch.zeros(5 * max(nr, 1), dtype=torch.int32, device=r.device)
        b.samp_greedy = True
        b.h_tokens = [torch.zeros(max(nr, 1), dtype=torch.int32).pin_memory() for _ in range(2)]
        b.h_status = [torch.zeros(1, dtype=torch.int32).pin_memory() for _ in range(2)]
        b.events = [torch.cuda.Event() for _ in range(2)]
        b.turn, b.by_length = 0, None
        b.lanes = [None] * n
        h = b.meta_host.numpy()
        b.starts = []
        pos = 0
        for i, ql in enumerate(q_lens):
            b.starts.append(pos)
            h[lay.positions + pos: lay.positions + pos + ql] = np.arange(ql)
            h[lay.token_seq + pos: lay.token_seq + pos + ql] = i
            h[lay.cu_q + i] = pos
            pos += ql
        h[lay.cu_q + n] = pos
        h[lay.seq_fresh: lay.seq_fresh + n] = 1            # the scratch state slot starts from zero, like a new request's
        h[lay.logits_rows: lay.logits_rows + nr] = rows
        # every table entry names the scratch page: whatever position is looked up, the page exists
        for off, w in zip(lay.tables, lay.widths):
            h[off: off + n * w] = SCRATCH_PAGE
        h[lay.updates] = 0
        b.meta_dev.copy_(b.meta_host)
        ctx = r.context_from_layout(lay, b.meta_dev, list(q_lens), [0] * n)
        ctx.logits_rows = ctx.logits_rows[:nr]
        ctx.workspace = self.shape_workspace
        ctx.max_kv_len = r.max_model_len      # launch shapes must not depend on the requests
        ctx.captured = True
        ctx.key_share_level = level           # ... except by the context's coarse level, which is part of the key
        ws_before = self.shape_workspace.version
        side = torch.cuda.Stream(device=r.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._apply_updates(b)
            logits = r.model.forward(ctx)     # sizes the scratch buffers; nothing may be allocated while capturing
            if nr:
                self._sample_rows(b, logits, nr)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(r.device)
        if self.shape_workspace.version != ws_before and self.shapes:
            self.shapes.clear()               # a scratch buffer moved: graphs that hold its old address are void
        b.graph = torch.cuda.CUDAGraph()
        before = K.LAUNCHES
        with _Capture(b.graph):
            self._apply_updates(b)
            b.logits = r.model.forward(ctx)
            if nr:
                self._sample_rows(b, b.logits, nr)
        b.launches = K.LAUNCHES - before
        self.shape_captures += 1
        return b

    def _sample_rows(self, b: _Bucket, logits: torch.Tensor, nr: int) -> None:
        d = b.samp_dev
        K.sample(logits, b.tokens[:nr], d[4 * nr:].view(torch.float32), d[:2 * nr].view(torch.int64),
                 d[2 * nr: 4 * nr].view(torch.int64))

    def _fill_shape(self, b: _Bucket, entries: Sequence[StepEntry]) -> None:
        r, lay = self.runner, b.layout
        h = b.meta_host.numpy()

        def put(off, values):
            h[off: off + len(values)] = values
            b.changes.append((off, values))
        for i, e in enumerate(entries):
            rc, ql, at = e.cache, b.q_lens[i], b.starts[i]
            cl = rc.num_tokens
            toks = np.asarray(e.tokens, dtype=np.int64)
            if toks.min() < 0 or toks.max() >= r.vocab_size:
                raise ValueError(f"request {rc.request_id!r}: token id outside the vocabulary")
            if cl + ql > r.max_model_len:
                raise ValueError(f"request {rc.request_id!r} exceeds max_model_len")
            h[lay.token_ids + at: lay.token_ids + at + ql] = toks
            h[lay.positions + at: lay.positions + at + ql] = np.arange(cl, cl + ql)
            h[lay.ctx_lens + i] = cl
            h[lay.seq_fresh + i] = 1 if rc.fresh else 0
            h[lay.state_slots + i] = rc.state_slot
            old = b.lanes[i]
            same = old is not None and old[0] == rc.serial
            lens = []
            for g, table in enumerate(rc.tables):
                if len(table) < -(-(cl + ql) // r.cache.groups[g].block_size):
                    raise OutOfPages(f"request {rc.request_id!r} lacks pages in group {g} for this step")
                row = lay.tables[g] + i * lay.widths[g]
                if same and old[2][g] == rc.first_live[g] and old[1][g] <= len(table):
                    if old[1][g] < len(table):
                        put(row + old[1][g], table[old[1][g]:])
                else:
                    put(row, list(table))
                lens.append(len(table))
            b.lanes[i] = (rc.serial, lens, list(rc.first_live))

    def run_shape(self, plan, entries: Sequence[StepEntry], sampling=None):
        """Run one step of a captured shape (capturing it first if need be).  ``sampling``: per wanted
        row (temperature, seed, counter) or None for arg-max everywhere.  Returns (tokens sampled at the
        wanted rows in the caller's order, device status), or (None, 0) without a wait when nothing is
        wanted."""
        order, key = plan
        b = self.shapes.get(key)
        if b is None:
            if len(self.shapes) >= self.MAX_SHAPES:
                self.shapes.popitem(last=False)
            b = self.shapes[key] = self._prepare_shape(key)
        self.shapes.move_to_end(key)
        ordered = [entries[i] for i in order]
        self._fill_shape(b, ordered)
        nr = len(b.rows)
        k = b.turn
        b.turn ^= 1
        if b.stage_events[k] is not None:
            b.stage_events[k].synchronize()        # the upload that last read this pinned buffer has happened
        else:
            b.stage_events[k] = torch.cuda.Event()
        if nr:
            size_was, b.size = b.size, nr          # the sampling buffer has one lane per wanted row
            self._upload_sampling(b, k, sampling)
            b.size = size_was
        stage = b.meta_stage[k]
        upto = b.layout.head_size if self._write_updates(b) else b.layout.size
        self.full_uploads += upto == b.layout.size
        stage[:upto].copy_(b.meta_host[:upto])
        b.meta_dev[:upto].copy_(stage[:upto], non_blocking=True)
        b.stage_events[k].record()
        self.h2d_bytes += 4 * upto
        b.graph.replay()
        self.shape_replays += 1
        self.kernel_launches += b.launches
        for e in ordered:
            self.runner.cache.advance(e.cache, len(e.tokens))
        self.runner.steps_run += 1
        if not nr:
            return None, 0
        b.h_tokens[k][:nr].copy_(b.tokens[:nr], non_blocking=True)
        b.h_status[k].copy_(self.runner.status, non_blocking=True)
        b.events[k].record()
        b.events[k].synchronize()
        return b.h_tokens[k][:nr].tolist(), int(b.h_status[k][0])

    @staticmethod
    def collect(step: LaunchedStep) -> Optional[List[int]]:
        """Wait for a launched step; its sampled tokens (None if they were not asked for)."""
        if step.event is None:
            return None
        step.event.synchronize()
        step.status_code = int(step.h_status[0])
        return step.h_tokens[:step.n].tolist()

    def run(self, entries: Sequence[StepEntry], want_tokens: bool = True, sampling=None
            ) -> Tuple[torch.Tensor, Optional[List[int]]]:
        """One decode step for ``entries`` (one token each).  Returns the logits
        [n, vocab] (valid until the next replay of this bucket) and, when asked,
        the sampled tokens already copied to the host."""
        step = self.launch(entries, want_tokens, sampling=sampling)
        return step.logits, self.collect(step)
