"""The engine loop: schedule, step, sample, finish; and its public faces.

``Engine`` follows the reference's class of that name (include/firefly/engine.h:16-73,
src/engine.cc): ``async_generate(id, input_ids, max_tokens)`` queues a request
from any thread, ``start()`` / ``stop()`` run the loop in a background thread and
results arrive on a ``ResultQueue`` as (request id, new token ids, is_finished)
— token ids where the reference pushes text, since text is outside this engine.
``max_prefill_chunk_size`` has the reference's meaning; left unset it is the reference's 256 while
some request is decoding and the step's whole token budget while none is.
One iteration is ``Engine.step()``: the scheduler picks portions and decode
tokens, the step function runs them as one batch, the sampler picks next tokens.

Decode steps that run from a CUDA graph are overlapped with the host's work
(``overlap_decode``): while step n runs, step n+1 for the same requests is put on
the stream, its input tokens copied on the device from step n's output (the arg-max
or the temperature draw: the sampler is part of the graph), and only then are step
n's tokens read.  The device never waits for the scheduler.  A step
is launched ahead only when no request of the batch can end by length at step n,
none waits for admission and every request gets its next page; a request that ends
at step n by an end-of-sequence token has one more token computed, which is dropped.
"""
from __future__ import annotations

import json
import os
import queue
import threading
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager, plan_groups
from ..config.base import ModelConfig
from ..models.decoder import DecoderModel
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .loading import load_model, random_model
from .request import GenerationRequest, RequestStatus
from .runner import ModelRunner, StepEntry, status_text
from .scheduler import Scheduler


@dataclass
class StepOutput:
    request_id: str
    new_tokens: List[int]
    is_finished: bool
    finish_reason: Optional[str] = None


class ResultQueue:
    """Thread-safe queue of ``StepOutput`` (the reference's ResultQueue carries
    {req_id, text, is_finished}, include/firefly/queue.h:11-57)."""

    def __init__(self):
        self._q: "queue.Queue[StepOutput]" = queue.Queue()

    def push(self, item: StepOutput) -> None:
        self._q.put(item)

    def pop(self, timeout: Optional[float] = None) -> Optional[StepOutput]:
        try:
            return self._q.get(timeout=timeout)
        except queue.Empty:
            return None


@dataclass
class _InFlight:
    """A decode step on the stream whose tokens the host has not read yet."""
    step: object                            # graphs.LaunchedStep
    requests: List[GenerationRequest]
    dropped: List[bool]                     # per lane: the request ended before this step's token


DEFAULT_PREFILL_CHUNK = 256      # the reference's default (include/firefly/engine.h:20, src/server.cu:84)


@dataclass
class EngineOptions:
    # the reference's --max-prefill-chunk-size: most prompt tokens of one request in one step.  None: the
    # reference's 256 while some request is decoding (a portion bounds what a prompt adds to their steps),
    # and as much as the step's token budget allows while none is (then portions only cost)
    max_prefill_chunk_size: Optional[int] = None
    max_batch_size_limit: int = 64          # most active requests (reference: 64)
    max_num_batched_tokens: int = 8192      # tokens of one step, all requests together
    kv_block_size: int = 16                 # tokens per cache page (reference: 16)
    num_kv_blocks: Optional[int] = None     # pages per cache group; None: from memory_fraction
    memory_fraction: float = 0.90           # of free device memory, for pages (reference: 0.90)
    max_model_len: Optional[int] = None     # None: the model's max positions
    eos_token_ids: Optional[Sequence[int]] = None   # None: config.json's eos_token_id, if any
    use_cuda_graphs: bool = True
    capture_repeating_steps: bool = True    # steps of other shapes (prompt portions) are captured when their shape comes again
    overlap_decode: bool = True             # launch the next greedy decode step before this one's tokens are read
    graph_batch_sizes: Sequence[int] = (1, 2, 4, 8, 16, 32, 64)   # reference: engine.h:72


class Engine:
    def __init__(self, model: DecoderModel, config: Optional[ModelConfig] = None,
                 result_queue: Optional[ResultQueue] = None, max_prefill_chunk_size: Optional[int] = None,
                 options: Optional[EngineOptions] = None, raw_config: Optional[dict] = None,
                 runner=None, sampler=None):
        """``runner`` / ``sampler``: stand-ins for the step function and the sampler (tests of the
        loop's decisions that need no device); by default the engine makes its own."""
        opts = options or EngineOptions()
        if options is None:
            opts.max_prefill_chunk_size = max_prefill_chunk_size
        self.options = opts
        self.prefill_chunk = opts.max_prefill_chunk_size or DEFAULT_PREFILL_CHUNK
        self.model = model
        self.config = config
        self.result_queue = result_queue
        self.device = model.rt.device
        max_len = opts.max_model_len or model.spec.max_positions
        max_len = min(max_len, model.spec.max_positions)
        slot_specs = model.cache_slot_specs()
        counts, capacity = self._size_cache_groups(slot_specs, opts, max_len)
        self.cache = CacheManager(slot_specs, block_size=opts.kv_block_size, num_blocks=counts,
                                  max_requests=opts.max_batch_size_limit)
        self.cache.allocate_storage(model.rt.dtype, self.device)
        # no request can be longer than what the groups that keep every key can hold
        self.max_model_len = max_len if capacity is None else min(max_len, capacity)
        self.runner = runner if runner is not None else ModelRunner(
            model, self.cache, max_model_len=self.max_model_len,
            max_batched_tokens=opts.max_num_batched_tokens, max_seqs=opts.max_batch_size_limit)
        eos = opts.eos_token_ids
        if eos is None:
            e = (raw_config or {}).get("eos_token_id")
            eos = [] if e is None else ([int(x) for x in e] if isinstance(e, list) else [int(e)])
        self.scheduler = Scheduler(self.cache, max_batch_size_limit=opts.max_batch_size_limit,
                                   max_prefill_chunk_size=self.prefill_chunk,
                                   max_num_batched_tokens=opts.max_num_batched_tokens,
                                   max_model_len=self.max_model_len, eos_token_ids=eos,
                                   whole_prompts_when_idle=opts.max_prefill_chunk_size is None
                                   and not any(g.spec.window is not None for g in self.cache.groups))
        self.sampler = sampler if sampler is not None else Sampler(self.device, opts.max_batch_size_limit)
        self.graphs = None
        # a model with a part that reads device values on the host runs launch by launch
        if opts.use_cuda_graphs and not getattr(model, "host_synchronous", False):
            from .graphs import DecodeGraphs
            self.graphs = DecodeGraphs(self.runner, opts.graph_batch_sizes)
        self._inbox: "queue.Queue[GenerationRequest]" = queue.Queue()
        self._thread: Optional[threading.Thread] = None
        self._running = False
        self.requests: Dict[str, GenerationRequest] = {}
        self.stats = {"steps": 0, "graph_steps": 0, "tokens": 0, "preemptions": 0, "launched_ahead": 0,
                      "dropped_tokens": 0, "device_errors": 0}
        self._inflight: Optional[_InFlight] = None
        self._loop_error: Optional[BaseException] = None

    def _size_cache_groups(self, slot_specs, opts: EngineOptions, max_len: int):
        """Pages per cache group.  Groups that keep every key get room for the same number of tokens:
        ``num_kv_blocks`` pages of ``kv_block_size`` if given, else what ``memory_fraction`` of the free
        device memory holds (after the step's scratch memory), at most ``max_batch_size_limit`` requests
        of ``max_len`` tokens.  A group whose layers read a window only needs, per request, the pages of
        its window plus one portion; it gets no more than that.  Returns (counts, tokens the
        every-key groups hold, or None if there is no such group)."""
        groups = plan_groups(slot_specs, opts.kv_block_size)
        if not groups:
            return [], None
        es = torch.empty((), dtype=self.model.rt.dtype).element_size()
        per_token = [len(slots) * 2 * sp.num_kv_heads * sp.head_dim * es for sp, slots, _ in groups]
        most = opts.max_batch_size_limit * max_len

        def window_pages(sp, bs):
            per_request = -(-(sp.window + self.prefill_chunk) // bs) + 2
            return opts.max_batch_size_limit * min(per_request, -(-max_len // bs) + 1)
        if opts.num_kv_blocks is not None:
            tokens = opts.num_kv_blocks * opts.kv_block_size
        else:
            free, _ = torch.cuda.mem_get_info(self.device)
            budget = int(max(0, free - self._scratch_estimate(opts)) * opts.memory_fraction)
            for (sp, _, bs), pt in zip(groups, per_token):
                if sp.window is not None:
                    budget -= window_pages(sp, bs) * bs * pt
            full = sum(pt for (sp, _, _), pt in zip(groups, per_token) if sp.window is None)
            tokens = min(most, max(0, budget) // max(1, full)) if full else most
        counts = []
        for sp, _, bs in groups:
            n = tokens // bs
            if sp.window is not None:
                n = min(n, window_pages(sp, bs))
            counts.append(int(n))
        if min(counts) < 1:
            raise RuntimeError("no memory left for cache pages")
        has_full = any(sp.window is None for sp, _, _ in groups)
        capacity = min(c * bs for c, (sp, _, bs) in zip(counts, groups) if sp.window is None) if has_full else None
        return counts, capacity

    def _scratch_estimate(self, opts: EngineOptions) -> int:
        """Bytes to leave for the scratch memory of the largest step and the library's own: activations
        of ``max_num_batched_tokens`` tokens (about 64 bytes per token and hidden unit covers the
        residual, the projections and a feed-forward four times as wide), logits of every request in
        32-bit twice (eager and captured), and half a gigabyte for the matrix library's workspaces."""
        spec = self.model.spec
        return (opts.max_num_batched_tokens * spec.hidden_size * 64
                + 2 * opts.max_batch_size_limit * spec.vocab_size * 4 + (512 << 20))

    # ---- the reference's interface ----------------------------------------------
    def async_generate(self, id: str, input_ids: Sequence[int], max_tokens: int = 512,
                       sampling: Optional[SamplingParams] = None) -> None:
        """Queue a request; thread-safe."""
        sp = sampling or SamplingParams(max_tokens=max_tokens)
        self._inbox.put(GenerationRequest(str(id), [int(t) for t in input_ids], sp))

    def start(self) -> None:
        if self._thread is not None:
            return
        self._running = True
        self._thread = threading.Thread(target=self._loop, name="firefly-engine", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        """Stop the loop and wait for it.  An exception that ended the loop is raised here (every
        request that was live then has already been finished with an error on the result queue)."""
        self._running = False
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        err, self._loop_error = self._loop_error, None
        if err is not None:
            raise RuntimeError(f"the engine loop ended with an error: {err}") from err

    def _push(self, out: StepOutput) -> None:
        if self.result_queue is not None:
            self.result_queue.push(out)

    def _loop(self) -> None:
        try:
            if self.device.type == "cuda":
                torch.cuda.set_device(self.device)
            while self._running:
                self._drain_inbox()
                if not self.scheduler.has_unfinished_requests() and self._inflight is None:
                    time.sleep(0.0005)
                    continue
                for out in self.step():
                    self._push(out)
            for out in self.drain():                     # a step may still be on the stream
                self._push(out)
        except BaseException as e:  # noqa: BLE001 - whatever it is, nobody may be left waiting
            self._loop_error = e
            self._running = False
            self._fail_all(f"error: engine loop failed: {type(e).__name__}: {e}")

    def _fail_all(self, reason: str) -> None:
        """Finish every request the engine knows of (running, waiting, not yet admitted) with
        ``reason``, so that no caller waits on the result queue for ever."""
        self._inflight = None
        live = list(self.scheduler.active_requests) + list(self.scheduler.pending_requests)
        while True:
            try:
                live.append(self._inbox.get_nowait())
            except queue.Empty:
                break
        for req in live:
            try:
                self.scheduler.finish_request(req, reason)
            except Exception:  # noqa: BLE001 - the bookkeeping itself may be what failed
                req.status, req.finish_reason = RequestStatus.FINISHED, reason
            self.requests.pop(req.id, None)
            self._push(StepOutput(req.id, [], True, reason))

    def _device_error(self, code: int, requests: Sequence[GenerationRequest]) -> List[StepOutput]:
        """A kernel of the step that ``requests`` were in raised the device status word: end them
        with an error (which request it was cannot be told), clear the word, launch nothing ahead."""
        reason = f"error: device status {code}: {status_text(code)}"
        self.stats["device_errors"] += 1
        self.runner.clear_status()
        outs = []
        for req in requests:
            if req.status is RequestStatus.FINISHED:
                continue
            self.scheduler.finish_request(req, reason)
            self.requests.pop(req.id, None)
            outs.append(StepOutput(req.id, [], True, reason))
        return outs

    def _drain_inbox(self) -> None:
        while True:
            try:
                req = self._inbox.get_nowait()
            except queue.Empty:
                return
            try:
                self.add_request(req)
            except ValueError as e:
                req.status = RequestStatus.FINISHED
                req.finish_reason = f"error: {e}"
                if self.result_queue is not None:
                    self.result_queue.push(StepOutput(req.id, [], True, req.finish_reason))

    # ---- synchronous core ----------------------------------------------------------
    def add_request(self, req: GenerationRequest) -> None:
        V = self.model.spec.vocab_size
        if any(t < 0 or t >= V for t in req.prompt_tokens):
            raise ValueError(f"request {req.id!r}: token id outside [0, {V})")
        self.scheduler.add_request(req)
        self.requests[req.id] = req

    def has_unfinished_requests(self) -> bool:
        return (self.scheduler.has_unfinished_requests() or not self._inbox.empty()
                or self._inflight is not None)

    # ---- decode steps launched ahead ---------------------------------------------------
    def _can_launch_ahead(self, cur: _InFlight) -> bool:
        """May the step after ``cur`` go on the stream before ``cur``'s tokens are known?"""
        sch = self.scheduler
        if sch.pending_requests or not self._inbox.empty() or any(cur.dropped):
            return False
        if len(sch.active_requests) != len(cur.requests) or \
                any(a is not b for a, b in zip(sch.active_requests, cur.requests)):
            return False
        for req in cur.requests:
            # cur's token makes generated+1 and total+1; the request must go on after it
            if len(req.generated_tokens) + 1 >= req.max_tokens or req.get_total_len() + 1 >= self.max_model_len:
                return False
        # the next page of every request, all or nothing
        if not all(self.cache.can_grow(req.cache, req.cache.num_tokens + 1) for req in cur.requests):
            return False
        need = [sum(self.cache.pages_needed(req.cache, req.cache.num_tokens + 1)[g] for req in cur.requests)
                for g in range(len(self.cache.groups))]
        return all(grp.allocator.num_free >= n for grp, n in zip(self.cache.groups, need))

    def _launch_ahead(self, cur: _InFlight) -> _InFlight:
        for req in cur.requests:
            ok = self.cache.grow(req.cache, req.cache.num_tokens + 1)
            assert ok
        entries = [StepEntry(req.cache, [0], [0]) for req in cur.requests]     # ids come from cur on the device
        # cur's token is not recorded yet: the step after it draws with the next counter
        step = self.graphs.launch(entries, want_tokens=True, tokens_from_last_replay=True,
                                  sampling=self._lane_sampling(cur.requests, ahead=1))
        self.stats["graph_steps"] += 1
        self.stats["launched_ahead"] += 1
        return _InFlight(step, list(cur.requests), [False] * len(cur.requests))

    @staticmethod
    def _lane_sampling(requests, ahead: int = 0):
        """Per request (temperature, seed, counter of the draw); None when all are greedy."""
        if all(r.sampling.temperature <= 0 for r in requests):
            return None
        return [(r.sampling.temperature, r.sampling.seed, len(r.generated_tokens) + ahead) for r in requests]

    def drain(self) -> List[StepOutput]:
        """Read the tokens of a step that is still on the stream, launching nothing new."""
        return self._finish_inflight(launch_next=False) if self._inflight is not None else []

    def _finish_inflight(self, launch_next: bool = True) -> List[StepOutput]:
        """Read the tokens of the step on the stream, after putting the next one there if that
        is allowed."""
        cur = self._inflight
        nxt = self._launch_ahead(cur) if launch_next and self._can_launch_ahead(cur) else None
        tokens = self.graphs.collect(cur.step)
        outputs: List[StepOutput] = []
        self.stats["steps"] += 1
        if cur.step.status_code:
            if nxt is not None:
                self.graphs.collect(nxt.step)         # it ran on the same, possibly damaged, cache: dropped
            self._inflight = None
            live = [r for r, dropped in zip(cur.requests, cur.dropped) if not dropped]
            return self._device_error(cur.step.status_code, live)
        for lane, (req, tok) in enumerate(zip(cur.requests, tokens)):
            if cur.dropped[lane]:
                self.stats["dropped_tokens"] += 1
                continue
            self.stats["tokens"] += 1
            done = self.scheduler.append_token(req, tok)
            outputs.append(StepOutput(req.id, [int(tok)], done, req.finish_reason))
            if done:
                self.requests.pop(req.id, None)
                if nxt is not None:
                    nxt.dropped[lane] = True          # its pages are free again; the stream keeps the order
        self._inflight = nxt
        return outputs

    def step(self) -> List[StepOutput]:
        """One iteration: returns what each affected request produced."""
        if self._inflight is not None:
            return self._finish_inflight()
        batch = self.scheduler.step()
        outputs: List[StepOutput] = []
        for req in batch.failed:
            outputs.append(StepOutput(req.id, [], True, req.finish_reason))
            self.requests.pop(req.id, None)
        self.stats["preemptions"] += len(batch.preempted)
        if not batch.items:
            return outputs
        sampling_items = [it for it in batch.items if it.samples]
        entries = [StepEntry(it.request.cache,
                             it.request.tokens_between(it.start, it.start + it.num_tokens),
                             [it.num_tokens - 1] if it.samples else []) for it in batch.items]
        params = [it.request.sampling for it in sampling_items]
        counters = [len(it.request.generated_tokens) for it in sampling_items]
        tokens = None
        code = 0
        if (self.graphs is not None and len(sampling_items) == len(batch.items)
                and all(it.num_tokens == 1 for it in batch.items)
                and self.graphs.supports(len(entries))):
            reqs = [it.request for it in batch.items]
            lanes = self._lane_sampling(reqs)
            self.stats["graph_steps"] += 1
            if self.options.overlap_decode:
                self._inflight = _InFlight(self.graphs.launch(entries, want_tokens=True, sampling=lanes),
                                           reqs, [False] * len(entries))
                return outputs + self._finish_inflight()
            logits, tokens = self.graphs.run(entries, want_tokens=True, sampling=lanes)
            status = self.runner.queue_status_read()
            code = status.code()
        else:
            plan = self.graphs.shape_ready(entries) \
                if self.graphs is not None and self.options.capture_repeating_steps else None
            if plan is not None:
                # a shape that came before: one replay instead of some hundred launches
                lanes = None if all(p.temperature <= 0 for p in params) else \
                    [(p.temperature, p.seed, c) for p, c in zip(params, counters)]
                tokens, code = self.graphs.run_shape(plan, entries, lanes)
                tokens = tokens or []
                self.stats["graph_steps"] += 1
            else:
                logits = self.runner.step(entries)
                # the status word is copied behind the step; reading the tokens (below) waits past it
                status = self.runner.queue_status_read()
                tokens = self.sampler.sample(logits, params, counters)
                if sampling_items or self._status_due():
                    code = status.code()
        if code:
            return outputs + self._device_error(code, [it.request for it in batch.items])
        self.stats["steps"] += 1
        self.stats["tokens"] += batch.num_tokens
        for it, tok in zip(sampling_items, tokens):
            done = self.scheduler.append_token(it.request, tok)
            outputs.append(StepOutput(it.request.id, [int(tok)], done, it.request.finish_reason))
            if done:
                self.requests.pop(it.request.id, None)
        return outputs


    STATUS_EVERY = 16     # steps without any sampled token (prompt portions only) between two looks at the status

    def _status_due(self) -> bool:
        self._unchecked = getattr(self, "_unchecked", 0) + 1
        if self._unchecked >= self.STATUS_EVERY:
            self._unchecked = 0
            return True
        return False


class LLM:
    """The Python entry point: ids in, ids out.

        llm = LLM("/path/to/model", dtype="bfloat16")
        outs = llm.generate([[1, 2, 3], [4, 5]], max_tokens=16)
    """

    def __init__(self, model, *, dtype="bfloat16", device="cuda:0", seed: int = 0, weight_dtype: str = "keep",
                 max_prefill_chunk_size: Optional[int] = None, **options):
        """``model``: a folder with config.json and model.safetensors, or a typed
        configuration (random weights drawn from ``seed``).  ``weight_dtype``: "keep" leaves a
        tensor stored in 32-bit as it is, "engine" narrows it to the engine's type on the device."""
        raw = None
        if isinstance(model, (str, os.PathLike)):
            self.model, self.config = load_model(str(model), dtype=dtype, device=device, weight_dtype=weight_dtype)
            with open(os.path.join(str(model), "config.json")) as fh:
                raw = json.load(fh)
        elif isinstance(model, ModelConfig):
            self.config = model
            self.model = random_model(model, seed, dtype=dtype, device=device)
        else:
            raise TypeError("model must be a folder or a ModelConfig")
        opts = EngineOptions(max_prefill_chunk_size=max_prefill_chunk_size, **options)
        self.engine = Engine(self.model, self.config, options=opts, raw_config=raw)
        self._next_id = 0

    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: int = 512, temperature: float = 0.0,
                 seed: int = 0, ignore_eos: bool = False,
                 sampling: Optional[Sequence[SamplingParams]] = None) -> List[List[int]]:
        """Generate for every prompt (lists of token ids); returns the new token
        ids of each, in order."""
        reqs = []
        for i, p in enumerate(prompts):
            sp = sampling[i] if sampling is not None else SamplingParams(
                temperature=temperature, seed=seed + i, max_tokens=max_tokens, ignore_eos=ignore_eos)
            req = GenerationRequest(f"gen-{self._next_id}", [int(t) for t in p], sp)
            self._next_id += 1
            self.engine.add_request(req)
            reqs.append(req)
        while self.engine.has_unfinished_requests():
            self.engine.step()
        self.engine.runner.check_status()
        for r in reqs:
            if r.finish_reason and r.finish_reason.startswith("error"):
                raise RuntimeError(f"request {r.id}: {r.finish_reason}")
        return [list(r.generated_tokens) for r in reqs]
