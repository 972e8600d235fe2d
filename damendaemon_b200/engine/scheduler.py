"""The scheduler above the step function: admits requests, cuts prompts into portions under
a token budget, decodes, finishes and frees.

Decisions (the reference's, where it has them):
* Admission is first-come first-served. A request is admitted when a request slot is free
  and the cache can promise pages for its prompt plus max_tokens; if it cannot, the request
  waits at the head of the queue and nothing behind it overtakes (damendaemon/scheduler.py:763-780).
  A request that could never fit the whole pool fails at once (damendaemon/paged.py:47-48).
  So an admitted request never runs out of pages in the middle of decoding; nothing is ever
  evicted or swapped (the reference has no preemption either).
* Without reservations (``reserve=False``) pages are claimed step by step. When a step does not
  fit, the youngest admitted requests are left out of it until it does; if not even the oldest
  request can take its next token, the youngest live request fails with 'cache_full' and its
  pages go back, so the others can go on.
* Every step holds all decoding requests (one token each) and fills the rest of the token
  budget with prompt portions of the admitted requests in admission order, each at most
  ``chunk_size`` tokens: one call of the step function, where the reference runs at most one
  chunk of one request and then a separate decode batch (damendaemon/scheduler.py:680-722,827-873).
  A prompt that is cut is cut at a multiple of ``engine.portion_multiple`` tokens where the portion
  is longer than that (the key block of the engine's prompt attention, 1 if it has none).
* prompt + max_tokens must fit the context (damendaemon/prompts.py:4-9); with
  ``length_policy='clamp'`` max_tokens is cut to what fits instead.
* A request ends on an end-of-sequence token (unless ignore_eos), at max_tokens ('length'),
  or at the model's last position. Its pages are given back before its last event is handed
  out (damendaemon/scheduler.py:869-873).
* A step that raises fails the requests in it and gives back their pages; the others go on
  (damendaemon/scheduler.py:812-818,881-895).
* Running ahead. While only decoding requests are live, nobody who waits can be admitted and no
  request can end by length in the step at hand, the next decode step is launched before this step's tokens are
  read: the engine takes its token ids from the sampler's output on the device. The host's work
  for a step then runs beside the device's, not between two steps. Only an end-of-sequence token
  can end a request unforeseen; such a request took part in one step too many, whose row is
  dropped, and everything it held goes back as always. Needs a sampler with ``launch`` and
  ``read`` (the default has them) and page reservations; ``run_ahead=False`` switches it off.
  The reference's scheduler reads every step's tokens before it plans the next.
* A request can be withdrawn (``cancel``) while it waits, between two portions of its prompt, or while it
  decodes, also with a step launched ahead that still holds it (that step's row for it is dropped, as after an
  end-of-sequence token). What it holds, pages and promise, goes back before its last event is handed out; its
  finish reason is 'cancelled' (damendaemon/scheduler.py:856-862 frees a cancelled request's slot in the same turn).
* With ``queue_timeout`` (seconds) a request that has waited that long for its pages fails with
  'KV admission timeout' (damendaemon/scheduler.py:758-761); the ones behind it move up.
* ``max_context`` caps prompt + generated tokens below the model's positions (a runtime whose page pool was sized
  for a shorter context).
"""
from __future__ import annotations

import itertools
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Hashable, Optional

from ..cache import PageCapacityError
from ..sampling import Sampler, Sampling
from .engine import StepEntry

_ids = itertools.count()


@dataclass(eq=False)          # a request is itself, not its fields: membership tests must not compare prompts
class Request:
    prompt: list
    max_tokens: int = 128
    sampling: Sampling = field(default_factory=Sampling)
    ignore_eos: bool = False
    id: Hashable = None
    # filled in by the scheduler
    output: list = field(default_factory=list)
    fed: int = 0
    finish_reason: Optional[str] = None
    error: Optional[str] = None
    sampler: Optional[Sampler] = None
    submitted_at: float = 0.0
    first_token_at: Optional[float] = None
    finished_at: Optional[float] = None
    cancel_requested: bool = False

    def __post_init__(self):
        if self.id is None:
            self.id = f"request-{next(_ids)}"

    @property
    def finished(self):
        return self.finish_reason is not None


@dataclass
class TokenEvent:
    request: Request
    token: Optional[int]      # None for a request that ended without a token (an error)
    finished: bool


@dataclass
class _InFlight:
    """A step whose forward pass has been launched and whose tokens have not been handed out."""
    entries: list                      # (request, tokens, want)
    rows: list                         # the requests a token is sampled for, in the order of the logits
    logits: object = None              # set while the sampling has not been launched yet
    pending: object = None             # what sample_fn.launch returned
    tokens: Optional[list] = None      # set when the sampler is a plain function: already read


class Scheduler:
    def __init__(self, engine, *, token_budget=2048, chunk_size=0, max_live=None, reserve=True,
                 length_policy="reject", sample_fn=None, run_ahead=True, queue_timeout=None, max_context=None,
                 clock=time.monotonic):
        if token_budget <= 0:
            raise ValueError("token_budget must be positive")
        if chunk_size < 0:
            raise ValueError("chunk_size must be 0 (no limit below the budget) or positive")
        if length_policy not in ("reject", "clamp"):
            raise ValueError("length_policy must be 'reject' or 'clamp'")
        if queue_timeout is not None and not queue_timeout > 0:
            raise ValueError("queue_timeout must be positive seconds, or None for no limit")
        if max_context is not None and not 0 < max_context <= engine.max_context:
            raise ValueError(f"max_context must be between 1 and the model's {engine.max_context} positions")
        self.engine = engine
        self.max_context = max_context or engine.max_context
        self.queue_timeout = queue_timeout
        self.clock = clock
        self.token_budget = token_budget
        self.chunk_size = chunk_size or token_budget
        self.max_live = min(max_live or engine.cache.max_requests, engine.cache.max_requests)
        self.reserve = reserve
        self.length_policy = length_policy
        if sample_fn is None:
            from ..sampling import sample_rows as sample_fn
        self.portion_multiple = max(1, int(getattr(engine, "portion_multiple", 1)))
        self.sample_fn = sample_fn
        self._launch, self._read = getattr(sample_fn, "launch", None), getattr(sample_fn, "read", None)
        self.run_ahead = bool(run_ahead and reserve and self._launch and self._read
                              and getattr(engine, "accepts_device_ids", False))
        self._in_flight = None
        self.steps_ahead = 0     # steps whose forward pass was launched before the tokens of the step before were read
        self.waiting = deque()
        self._known = {}         # id -> request, from submit until its end (one dictionary lookup serves cancel)
        self.prefilling = []     # admitted, prompt not yet wholly in the cache; admission order
        self.decoding = []       # admitted, generating; admission order
        self.done = []
        self.steps = 0
        self.step_log = []       # (prompt tokens, decode tokens) of each step

    # ------------------------------------------------------------------ intake
    def submit(self, request: Request) -> Request:
        context, vocab = self.max_context, self.engine.spec.vocab_size
        if not isinstance(request.prompt, list) or not request.prompt or \
                any(type(t) is not int or not 0 <= t < vocab for t in request.prompt):
            raise ValueError("prompt must be a nonempty list of token ids inside the vocabulary")
        if type(request.max_tokens) is not int or request.max_tokens <= 0:
            raise ValueError("max_tokens must be a positive integer")
        if len(request.prompt) + request.max_tokens > context:
            if self.length_policy == "reject" or len(request.prompt) >= context:
                raise ValueError("prompt plus max_tokens exceeds configured context")
            request.max_tokens = context - len(request.prompt)
        request.sampler = Sampler(request.sampling)
        request.sampler.prepare(request.prompt, vocab)
        request.submitted_at = time.perf_counter()
        request.waiting_since = self.clock()
        if request.id in self._known:
            raise ValueError(f"a request with id {request.id!r} is already in the scheduler")
        self._known[request.id] = request
        self.waiting.append(request)
        return request

    def cancel(self, request) -> bool:
        """Withdraw a request (the object ``submit`` returned, or its id). It takes effect at the start of the next
        ``step()``: whatever the request holds goes back, and that step's events end with its terminal event
        (token None, finish reason 'cancelled'). Returns False if the request is unknown or has ended already.
        Setting the flag is all this does, so another thread may call it while ``step()`` runs."""
        known = self._known.get(request.id if isinstance(request, Request) else request)
        if known is None or known.finished or (isinstance(request, Request) and known is not request):
            return False
        known.cancel_requested = True
        return True

    def _withdraw(self, events):
        """Apply cancellations and the queue timeout; runs before anything else in a step."""
        for request in [r for r in self.live() if r.cancel_requested]:
            self._end(request, "cancelled", None, events)
        now = self.clock()
        for request in list(self.waiting):
            if request.cancel_requested:
                self.waiting.remove(request)
                self._end(request, "cancelled", None, events, release=False)
            elif self.queue_timeout is not None and now - request.waiting_since > self.queue_timeout:
                self.waiting.remove(request)
                self._end(request, "error", "KV admission timeout", events, release=False)

    @property
    def idle(self):
        return not (self.waiting or self.prefilling or self.decoding)

    def live(self):
        return self.prefilling + self.decoding

    # ------------------------------------------------------------------ decisions
    def _admit(self, events):
        while self.waiting and len(self.live()) < self.max_live:
            request = self.waiting[0]
            total = len(request.prompt) + request.max_tokens
            try:
                if self.reserve:
                    self.engine.reserve(request.id, total, min(self.chunk_size, self.token_budget))
                else:
                    self.engine.cache.admit(request.id)
            except PageCapacityError:
                break                                   # wait at the head of the queue; nobody overtakes
            except ValueError as error:                 # can never fit
                self.waiting.popleft()
                self._fail(request, str(error), events, release=False)
                continue
            self.waiting.popleft()
            self.prefilling.append(request)

    def plan(self):
        """The next step's entries as (request, tokens, want), decided from host state only."""
        entries, budget = [], self.token_budget
        for request in self.decoding:
            entries.append((request, [request.output[-1]], [0]))
            budget -= 1
        for request in self.prefilling:
            if budget <= 0:
                break
            n = min(len(request.prompt) - request.fed, self.chunk_size, budget)
            final = request.fed + n == len(request.prompt)
            if not final and n > self.portion_multiple:
                # a portion that is cut ends where the engine likes the next one to start (a key block of its prompt
                # attention): the next portion then reads whole blocks and needs no separate cache write
                n -= (request.fed + n) % self.portion_multiple
            entries.append((request, request.prompt[request.fed:request.fed + n], [n - 1] if final else []))
            budget -= n
        if not self.reserve:
            entries = self._fit(entries)
        return entries

    def _fit(self, entries):
        """Leave out the youngest requests until the cache can take the step."""
        cache = self.engine.cache
        order = {r.id: i for i, r in enumerate(sorted(self.live(), key=lambda r: r.submitted_at))}
        kept = sorted(entries, key=lambda e: order[e[0].id])
        while kept and not cache.can_extend([(r.id, cache.length[r.id] + len(t)) for r, t, _ in kept]):
            kept.pop()
        return [e for e in entries if any(e[0] is k[0] for k in kept)]

    # ------------------------------------------------------------------ one step
    def _forward(self, entries, events, device_ids=None):
        """Launch the step's forward pass and, unless the ids come from the device, its sampling.
        A step that raises fails its requests; returns None then."""
        try:
            step_entries = [StepEntry(r.id, tokens, want) for r, tokens, want in entries]
            if device_ids is None:
                logits = self.engine.step(step_entries)
            else:
                logits = self.engine.step(step_entries, device_ids=device_ids)
            flight = _InFlight(entries, [r for r, _, want in entries if want], logits=logits)
            if device_ids is None:
                self._sample(flight)
            return flight
        except Exception as error:      # the step failed: its requests fail, the others go on
            for request, _, _ in entries:
                if not request.finished:
                    self._fail(request, f"{type(error).__name__}: {error}", events)
            return None

    def _sample(self, flight):
        logits, flight.logits = flight.logits, None
        if not flight.rows:
            flight.tokens = []
        elif self._launch and self._read:
            flight.pending = self._launch(logits, [r.sampler for r in flight.rows])
        else:
            flight.tokens = self.sample_fn(logits, [r.sampler for r in flight.rows])

    def _may_run_ahead(self, flight):
        """Only decoding requests are live, all of them are in this step, nobody who waits can be admitted now
        (the caller has tried), and none of them can end by length with the token this step samples."""
        if not self.run_ahead or flight.pending is None or self.prefilling:
            return False
        if len(flight.rows) != len(self.decoding) or len(flight.entries) != len(flight.rows):
            return False
        for request in flight.rows:
            if request not in self.decoding or len(request.output) + 1 >= request.max_tokens or \
                    len(request.prompt) + len(request.output) + 1 >= self.max_context:
                return False
        return True

    def step(self):
        """Admit, run one step of the engine, sample, finish. Returns the TokenEvents of the step whose
        tokens it read: the one it launched, or the one a call before launched ahead."""
        events = []
        self._withdraw(events)
        flight, self._in_flight = self._in_flight, None
        if flight is not None and all(r.finished for r, _, _ in flight.entries):
            flight = None               # everybody the step launched ahead was for has been withdrawn
        if flight is None:
            self._admit(events)
            entries = self.plan()
            if not entries:
                if not self.reserve and self.live():
                    youngest = max(self.live(), key=lambda r: r.submitted_at)
                    self._fail(youngest, "cache_full", events)
                return events
            flight = self._forward(entries, events)
            if flight is None:
                return events
        ahead = None
        if self.waiting and self.run_ahead and flight.pending is not None:
            self._admit(events)         # whoever can come in now makes the next step a mixed one: no running ahead then
        if self._may_run_ahead(flight):
            # the token values are placeholders: the engine takes the ids from the sampler's output
            ahead = self._forward([(r, [0], [0]) for r in flight.rows], events, device_ids=flight.pending.ids)
        try:
            tokens = flight.tokens if flight.tokens is not None else self._read(flight.pending)
        except Exception as error:
            for request, _, _ in flight.entries:
                if not request.finished:
                    self._fail(request, f"{type(error).__name__}: {error}", events)
            return events               # a step launched ahead held the same requests: dropped with them
        self.steps += 1
        self.step_log.append((sum(len(t) for r, t, _ in flight.entries if r in self.prefilling),
                              sum(1 for r, _, _ in flight.entries if r in self.decoding)))
        now = time.perf_counter()
        for request, fed_tokens, _ in flight.entries:
            if request in self.prefilling:
                request.fed += len(fed_tokens)
        for request, token in zip(flight.rows, tokens):
            if request.finished:
                continue                # it ended in the step before this one, which had been launched already
            if request in self.prefilling:
                self.prefilling.remove(request)
                self.decoding.append(request)
                request.first_token_at = now
            request.output.append(token)
            request.sampler.observe(token)
            reason = None
            if not request.ignore_eos and token in self.engine.spec.eos_token_ids:
                reason = "stop"
            elif len(request.output) >= request.max_tokens:
                reason = "length"
            elif len(request.prompt) + len(request.output) >= self.max_context:
                reason = "length"
            if reason:
                self._finish(request, reason)
            events.append(TokenEvent(request, token, reason is not None))
        if ahead is not None and any(not r.finished for r in ahead.rows):
            try:
                self._sample(ahead)     # after this step's tokens were observed: penalties and draws are in order
                self._in_flight = ahead
                self.steps_ahead += 1
            except Exception as error:
                for request in ahead.rows:
                    if not request.finished:
                        self._fail(request, f"{type(error).__name__}: {error}", events)
        return events

    def _finish(self, request, reason):
        self.engine.finish(request.id)                  # pages go back before the last event is seen
        self._known.pop(request.id, None)
        request.finish_reason = reason
        request.finished_at = time.perf_counter()
        for group in (self.prefilling, self.decoding):
            if request in group:
                group.remove(request)
        self.done.append(request)

    def _fail(self, request, message, events, release=True):
        self._end(request, "error", message, events, release)

    def _end(self, request, reason, message, events, release=True):
        """End a request without a token: what it holds goes back first, then its terminal event is queued."""
        if release:
            self.engine.finish(request.id)
        self._known.pop(request.id, None)
        request.finish_reason, request.error = reason, message
        request.finished_at = time.perf_counter()
        for group in (self.prefilling, self.decoding):
            if request in group:
                group.remove(request)
        self.done.append(request)
        events.append(TokenEvent(request, None, True))

    def run(self):
        """Step until every submitted request has ended; yields TokenEvents."""
        while not self.idle:
            events = self.step()
            yield from events
            if not events and not self.live() and self.waiting:
                # nothing is live and the head of the queue still cannot be admitted: it never will be
                request = self.waiting.popleft()
                failed = []
                self._fail(request, "cache pages do not suffice for this request", failed, release=False)
                yield from failed
