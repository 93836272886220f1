"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes, finishes
and frees; and decides what happens when pages run out.

Every :meth:`Scheduler.step` plans one batch and runs it through the engine's one step function:

1. one decode row for every running request whose prompt is in the cache;
2. portions of the prompts of running requests, oldest first (portion = min(rest of the prompt, rest of
   the token budget, the chunk cap), cut down to the pages that are free);
3. newly admitted requests from the waiting queue, first come first served, while a state slot, pages
   and budget are left.

When the decode rows need more pages than are free, the most recently admitted running request is
*preempted*: its pages and slot are given back and it returns to the front of the waiting queue with
prompt := original prompt + tokens generated so far (recomputed on re-admission; its sampler, and so its
random stream, is kept, so the continuation is the same).  If the one remaining request still cannot get
a page, it is finished with reason ``context_full``.  Decisions depend on the order of arrival only.

The reference's scheduler lives in its server (``tick``, bin/rocm-inference-server:1818-1871): a FIFO
queue, a fixed pool of sequences each with a whole-context cache, a prefill chunk of ``--prefill-chunk``
tokens (default 512, :1648) per tick beside batched decoding, no token budget and no preemption; stop
reasons are those of src/inference.h:229-236.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence

from ..cache.pages import OutOfPages
from ..sampling.sampler import Sampler, SamplerParams

# stop reasons, named after src/inference.h:229-236
STOP_NONE, STOP_EOG, STOP_MAX_TOKENS, STOP_CALLBACK, STOP_CONTEXT_FULL, STOP_CANCELLED = (
    "none", "eog", "max_tokens", "callback", "context_full", "cancelled")


@dataclass
class Request:
    request_id: object
    prompt: List[int]
    params: SamplerParams = field(default_factory=SamplerParams.greedy)
    max_new_tokens: int = 256
    eos_ids: Sequence[int] = ()
    ignore_eos: bool = False
    on_token: Optional[Callable] = None          # called with (request, token); a true return stops
    # state
    output: List[int] = field(default_factory=list)
    status: str = "waiting"                      # waiting | running | finished
    stop_reason: str = STOP_NONE
    sampler: Optional[Sampler] = None
    admitted_at: int = -1                        # admission counter, for "most recently admitted"
    preemptions: int = 0

    def tokens(self) -> List[int]:
        return self.prompt + self.output


@dataclass
class StepEvent:
    request_id: object
    token: Optional[int]                         # the token emitted in this step, if any
    finished: bool = False
    stop_reason: str = STOP_NONE


@dataclass
class PlannedEntry:
    request: Request
    start: int                                   # first token (index into request.tokens()) fed in this step
    count: int
    samples: bool                                # the portion ends the known tokens: its last row is sampled


class Scheduler:
    def __init__(self, engine, *, max_batch_tokens: int = 2048, prefill_chunk: int = 512, max_running: Optional[int] = None,
                 n_ctx: Optional[int] = None, align_rows: Optional[int] = None):
        """``engine`` offers ``cache`` (a :class:`CacheManager`), ``step(entries)`` and ``sample(logits,
        samplers)``, as :class:`purhie_b200.engine.Engine` does.  ``align_rows`` (default: the engine's
        ``row_tile``, if it names one): a prompt portion that is a cut anyway is shortened so that the step's rows
        end on a multiple of it, because the products run in tiles of that many rows and a step of 544 rows costs
        what one of 768 does."""
        self.engine = engine
        self.align_rows = align_rows if align_rows is not None else getattr(engine, "row_tile", None)
        self.run_ahead = True                       # decode_ahead() may launch steps before the tokens of the last are read
        self.cache = engine.cache
        self.max_batch_tokens = max_batch_tokens
        self.prefill_chunk = prefill_chunk
        self.max_running = max_running if max_running is not None else self.cache.max_requests
        self.n_ctx = n_ctx if n_ctx is not None else getattr(engine, "max_position", 1 << 30)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: Dict[object, Request] = {}
        self._admissions = 0
        self.steps = 0
        self.preemptions = 0

    # ---- requests --------------------------------------------------------------------------------
    def add(self, request: Request) -> Request:
        if not request.prompt:
            raise ValueError("a request needs at least one prompt token")
        if request.sampler is None:
            request.sampler = Sampler(request.params)
            for t in request.prompt:
                request.sampler.accept(t)         # the penalty window covers the prompt (src/inference.cpp:2791-2792)
        request.status = "waiting"
        self.waiting.append(request)
        return request

    def cancel(self, request_id) -> bool:
        for r in list(self.waiting):
            if r.request_id == request_id:
                self.waiting.remove(r)
                self._finish(r, STOP_CANCELLED, live=False)
                return True
        for r in self.running:
            if r.request_id == request_id:
                self._finish(r, STOP_CANCELLED)
                return True
        return False

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- planning --------------------------------------------------------------------------------
    def _computed(self, r: Request) -> int:
        return self.cache.length(r.request_id)

    def _fits(self, r: Request, n_new: int, free: List[int]) -> bool:
        return all(n <= f for n, f in zip(self.cache.pages_needed(r.request_id, n_new), free))

    def _take(self, r: Request, n_new: int, free: List[int]) -> None:
        for i, n in enumerate(self.cache.pages_needed(r.request_id, n_new)):
            free[i] -= n

    def _largest_portion(self, r: Request, want: int, free: List[int]) -> int:
        """The most tokens <= want for which pages are free."""
        ps = self.cache.page_size
        rc = self.cache.requests[r.request_id]
        best = want
        for g, f in zip(self.cache.groups, free):
            room = (len(rc.tables[g.index]) + f) * ps - rc.length
            best = min(best, room)
        return max(best, 0)

    def _aligned(self, n: int, rest: int, used: int) -> int:
        """The portion of n tokens (of rest that the request still has) after ``used`` rows of the step: when the
        prompt goes on after it and the step would end past a multiple of align_rows, the portion ends there
        instead, unless that takes more than half of it."""
        a = self.align_rows
        if not a or n >= rest or used + n < a:
            return n
        over = (used + n) % a
        return n - over if over and n - over >= max(n // 2, 1) else n

    def _preempt(self, r: Request) -> None:
        self.cache.release(r.request_id)
        self.running.remove(r)
        r.status = "waiting"
        r.preemptions += 1
        self.preemptions += 1
        self.waiting.appendleft(r)

    def _finish(self, r: Request, reason: str, live: bool = True) -> None:
        if live:
            self.cache.release(r.request_id)
            self.running.remove(r)
        r.status = "finished"
        r.stop_reason = reason
        self.finished[r.request_id] = r

    def plan(self) -> List[PlannedEntry]:
        """Decide this step's batch.  May preempt, admit and finish requests; reserves nothing."""
        events_before = len(self.finished)
        while True:
            free = self.cache.free_pages()
            budget = self.max_batch_tokens
            plan: List[PlannedEntry] = []
            decoders = [r for r in self.running if len(r.tokens()) - self._computed(r) == 1 and r.output]
            # 1. decode rows; make room by preempting the newest running request
            need = [0] * len(free)
            for r in decoders:
                for i, n in enumerate(self.cache.pages_needed(r.request_id, 1)):
                    need[i] += n
            if any(n > f for n, f in zip(need, free)) or len(decoders) > budget:
                victim = max(self.running, key=lambda r: r.admitted_at)
                if len(self.running) == 1:
                    self._finish(victim, STOP_CONTEXT_FULL)
                else:
                    self._preempt(victim)
                continue
            for r in decoders:
                self._take(r, 1, free)
                plan.append(PlannedEntry(r, len(r.tokens()) - 1, 1, True))
                budget -= 1
            # 2. prompt portions of running requests, oldest admission first
            for r in sorted(self.running, key=lambda r: r.admitted_at):
                if r in decoders or budget <= 0:
                    continue
                rest = len(r.tokens()) - self._computed(r)
                n = self._largest_portion(r, min(rest, budget, self.prefill_chunk), free)
                if n <= 0:
                    continue
                n = self._aligned(n, rest, self.max_batch_tokens - budget)
                self._take(r, n, free)
                plan.append(PlannedEntry(r, self._computed(r), n, n == rest))
                budget -= n
            # 3. admissions
            while self.waiting and budget > 0 and len(self.running) < self.max_running and self.cache.slots.num_free > 0:
                r = self.waiting[0]
                total_pages = [g.allocator.num_pages for g in self.cache.groups]
                if any(n > t for n, t in zip(self.cache.pages_for_new_request(len(r.tokens()) + 1), total_pages)) \
                        or len(r.tokens()) + 1 > self.n_ctx:
                    # even an empty pool (or the context) cannot hold this request and one more token
                    self.waiting.popleft()
                    self._finish(r, STOP_CONTEXT_FULL, live=False)
                    continue
                rest = len(r.tokens())
                n = min(rest, budget, self.prefill_chunk)
                pages = -(-n // self.cache.page_size)
                if any(pages > f for f in free):
                    n = min(free) * self.cache.page_size if free else n
                    if n <= 0:
                        break
                n = self._aligned(n, rest, self.max_batch_tokens - budget)
                self.waiting.popleft()
                self.cache.add_request(r.request_id)
                r.status = "running"
                r.admitted_at = self._admissions
                self._admissions += 1
                self.running.append(r)
                self._take(r, n, free)
                plan.append(PlannedEntry(r, 0, n, n == rest))
                budget -= n
            if not plan and self.running:
                # nobody can move: the pages are spread over half-done prompts; make room for the oldest
                victim = max(self.running, key=lambda r: r.admitted_at)
                if len(self.running) == 1:
                    self._finish(victim, STOP_CONTEXT_FULL)
                else:
                    self._preempt(victim)
                continue
            return plan

    # ---- one step --------------------------------------------------------------------------------
    def step(self) -> List[StepEvent]:
        """Plan a batch, run it, sample, and finish what is done.  Returns what happened, in batch order
        (plus requests that the planning finished without running them)."""
        from .engine import StepEntry
        done_before = set(self.finished)
        plan = self.plan()
        events: List[StepEvent] = [StepEvent(rid, None, True, self.finished[rid].stop_reason)
                                   for rid in self.finished if rid not in done_before]
        if not plan:
            return events
        entries, samplers, sampled = [], [], []
        for p in plan:
            toks = p.request.tokens()[p.start:p.start + p.count]
            entries.append(StepEntry(p.request.request_id, toks, [p.count - 1] if p.samples else []))
            if p.samples:
                samplers.append(p.request.sampler)
                sampled.append(p.request)
        logits = self.engine.step(entries)
        self.steps += 1
        tokens = self.engine.sample(logits, samplers) if sampled else []
        for r, tok in zip(sampled, tokens):
            events.append(self._emit(r, int(tok)))
        return events

    def _emit(self, r: Request, tok: int) -> StepEvent:
        if not r.ignore_eos and tok in r.eos_ids:
            self._finish(r, STOP_EOG)                    # the end-of-generation token is not emitted
            return StepEvent(r.request_id, None, True, STOP_EOG)
        r.output.append(tok)
        r.sampler.accept(tok)
        stop = bool(r.on_token(r, tok)) if r.on_token else False
        if stop:
            reason = STOP_CALLBACK
        elif len(r.output) >= r.max_new_tokens:
            reason = STOP_MAX_TOKENS
        elif len(r.tokens()) >= self.n_ctx:
            reason = STOP_CONTEXT_FULL
        else:
            return StepEvent(r.request_id, tok)
        self._finish(r, reason)
        return StepEvent(r.request_id, tok, True, reason)

    def decode_ahead(self, max_steps: int = 1 << 30) -> int:
        """While nothing waits and every running request is decoding with a device sampler: decode steps each
        launched with the token ids the step before left on the device, the host reading them one step behind.
        The run ends when a request finishes (what the step in flight sampled for it is dropped; its pages are
        given back as for any finished request, and are not handed out again before a later step is launched
        behind the one in flight), when pages run out (the ordinary step then decides whom to preempt) or at the
        step before the first request's token budget or the context could end it.  Returns the number of steps
        run; 0: not applicable, take an ordinary step."""
        from .engine import StepEntry
        from ..cache.pages import OutOfPages
        run = list(self.running)
        as_graph = getattr(self.engine, "decodes_as_graph", None)
        if not self.run_ahead or as_graph is None or self.waiting or not run or len(run) > self.max_batch_tokens:
            return 0
        if any(len(r.tokens()) - self._computed(r) != 1 or not r.output for r in run):
            return 0
        modes = {r.sampler.device_mode() for r in run}
        if len(modes) != 1 or None in modes:
            return 0
        probe = [StepEntry(r.request_id, [0], [0]) for r in run]
        horizon = min(min(r.max_new_tokens - len(r.output), self.n_ctx - len(r.tokens())) for r in run)
        n = min(max_steps, horizon)
        if n < 2 or not as_graph(probe):
            return 0
        samplers = [r.sampler for r in run]
        prev, done = None, 0

        def settle(toks) -> bool:
            ended = False
            for r, tok in zip(run, toks):
                ended |= self._emit(r, int(tok)).finished
            return ended

        for step in range(n):
            entries = [StepEntry(r.request_id, [r.output[-1]], [0]) for r in run] if step == 0 else probe
            try:
                logits = self.engine.step(entries, device_tokens=prev.ids if prev is not None else None)
            except OutOfPages:
                break
            self.steps += 1
            done += 1
            pend = self.engine.sample_async(logits, samplers)
            if prev is not None and settle(prev.result()):
                # the batch changes: the step in flight stands for the requests that go on
                toks = pend.result()
                for r, tok in zip(run, toks):
                    if r.status == "running":
                        self._emit(r, int(tok))
                return done
            prev = pend
        if prev is not None:
            settle(prev.result())
        return done

    def run(self) -> Dict[object, Request]:
        """Step until nothing is waiting or running."""
        while self.has_work():
            if not self.decode_ahead():
                self.step()
        return self.finished
