"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes, finishes and frees.

Policy, after the reference's planner (src/Starlings.Roost.Engine/Scheduling/StepPlanner.cs):
  * admission refuses an empty prompt, max_tokens <= 0, a duplicate id, and a prompt that could never fit its
    pools even alone (:177-215);
  * waiting and running requests are one list in a total order: priority descending, deadline ascending
    (none last), arrival ascending (:563-575);
  * a plan takes requests in that order until the token budget (default 2048) or the row cap (default 64) is
    reached; each takes min(tokens it still has to run, budget left, the portion cap): one token for a request
    that decodes, the rest of its prompt for one that prefills; a cut prompt goes on in the next plan
    (:585-645); a row samples iff it reaches the request's last known token (:870);
  * pages are taken when a row is planned, never ahead (:741-751). When they run out: if the free pages plus
    the pages of later-ordered resident requests would suffice, those are preempted from the tail (a victim
    keeps its tokens, the generated ones too, loses its pages and is recomputed from position 0 later,
    :669-698,970-976); if not, nobody is preempted and the request is skipped in this plan (:623-632); if no
    row at all can be planned, the best-ranked stalled request is aborted (:316-336);
  * a request finishes on a stop token, at max_tokens, or when its context is full, and its pages are given
    back at once (steps are synchronous: no plan in flight still names them).
Plans are a function of the sequence of calls: no clock, no randomness, no hash-order iteration.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..cache.manager import CacheManager
from .request import Request, RequestError, TokenEvent


@dataclass
class SchedulerOptions:
    max_tokens_per_step: int = 2048
    max_sequences_per_step: int = 64
    max_chunk_tokens: int | None = None
    model_stop_token_ids: tuple = ()
    max_context: int | None = None      # the model's positions, when it bounds them


@dataclass
class Sequence:
    request: Request
    arrival: int
    tokens: list                        # prompt and generated tokens
    prompt_len: int
    computed: int = 0                   # tokens whose cache entries exist (after the plan in hand has run)
    generated: int = 0
    preemptions: int = 0
    finished: str | None = None

    @property
    def request_id(self):
        return self.request.request_id

    @property
    def resident(self) -> bool:
        return self.computed > 0


@dataclass
class PlannedRow:
    sequence: Sequence
    start: int
    count: int
    samples: bool

    @property
    def tokens(self) -> list:
        return self.sequence.tokens[self.start : self.start + self.count]


@dataclass
class StepPlan:
    rows: list = field(default_factory=list)
    preempted: list = field(default_factory=list)   # request ids preempted while this plan was made
    aborted: list = field(default_factory=list)     # TokenEvents of requests aborted because they can never fit

    @property
    def num_tokens(self) -> int:
        return sum(r.count for r in self.rows)


class Scheduler:
    def __init__(self, cache: CacheManager, options: SchedulerOptions | None = None):
        self.cache = cache
        self.options = options or SchedulerOptions()
        if self.options.max_tokens_per_step <= 0 or self.options.max_sequences_per_step <= 0:
            raise ValueError("the token budget and the row cap must be positive")
        self._seqs: list[Sequence] = []
        self._arrivals = 0
        self.preemption_count = 0

    # ------------------------------------------------------------------ admission
    def add(self, request: Request) -> Sequence:
        if not request.prompt_token_ids:
            raise RequestError("InvalidOption", "the prompt is empty")
        request.sampling.validate()
        if any(s.request_id == request.request_id for s in self._seqs):
            raise RequestError("InvalidOption", f"request id {request.request_id!r} is already live")
        n = len(request.prompt_token_ids)
        if n + 1 > self.cache.max_tokens_per_request():
            raise RequestError("PromptTooLong", f"a prompt of {n} tokens and one generated token need more pages than the pool has "
                                                f"({self.cache.max_tokens_per_request()} tokens)")
        if self.options.max_context is not None and n + 1 > self.options.max_context:
            raise RequestError("PromptTooLong", f"a prompt of {n} tokens leaves no room for a generated token in {self.options.max_context} positions")
        seq = Sequence(request=request, arrival=self._arrivals, tokens=list(request.prompt_token_ids), prompt_len=n)
        self._arrivals += 1
        self._seqs.append(seq)
        return seq

    def cancel(self, request_id) -> bool:
        for s in self._seqs:
            if s.request_id == request_id:
                self._remove(s)
                return True
        return False

    @property
    def unfinished(self) -> int:
        return len(self._seqs)

    def sequences(self) -> list[Sequence]:
        return list(self._seqs)

    # ------------------------------------------------------------------ planning
    @staticmethod
    def _order_key(s: Sequence):
        d = s.request.deadline
        return (-s.request.priority, d is None, d if d is not None else 0.0, s.arrival)

    def plan(self) -> StepPlan | None:
        """The next step's rows, or None when no request is live. A plan may come back with no rows only
        together with aborted requests."""
        plan = StepPlan()
        while self._seqs:
            stalled = self._build(plan)
            if plan.rows or stalled is None:
                break
            # nothing could be planned although requests are live: the best-ranked stalled one can never fit
            self._remove(stalled)
            stalled.finished = "aborted"
            plan.aborted.append(TokenEvent(stalled.request_id, None, "aborted"))
        if not plan.rows and not plan.aborted:
            return None
        return plan

    def _build(self, plan: StepPlan):
        order = sorted(self._seqs, key=self._order_key)
        budget = self.options.max_tokens_per_step
        stalled = None
        for i, s in enumerate(order):
            if len(plan.rows) >= self.options.max_sequences_per_step or budget <= 0:
                break
            remaining = len(s.tokens) - s.computed
            if remaining <= 0:
                continue  # waits for its sampled token
            n = min(remaining, budget)
            if self.options.max_chunk_tokens:
                n = min(n, self.options.max_chunk_tokens)
            if not self._reserve(s, n, order, i, plan):
                stalled = stalled or s
                continue
            plan.rows.append(PlannedRow(s, s.computed, n, samples=s.computed + n == len(s.tokens)))
            budget -= n
            s.computed += n
        return stalled

    def _reserve(self, s: Sequence, n: int, order: list, index: int, plan: StepPlan) -> bool:
        target = s.computed + n
        if self.cache.can_hold(s.request_id, target):
            self.cache.extend(s.request_id, target)
            return True
        # feasible with what later-ordered resident requests hold?
        planned = {r.sequence.request_id for r in plan.rows}
        victims = [v for v in order[index + 1 :] if v.request_id in self.cache and v.request_id not in planned]
        extra = [0] * len(self.cache.groups)
        for v in victims:
            for gi, h in enumerate(self.cache.held(v.request_id)):
                extra[gi] += h
        if not self.cache.can_hold(s.request_id, target, extra_free=extra):
            return False
        for v in reversed(victims):
            self._preempt(v)
            plan.preempted.append(v.request_id)
            if self.cache.can_hold(s.request_id, target):
                break
        self.cache.extend(s.request_id, target)
        return True

    def rollback(self, plan: StepPlan) -> None:
        """The plan's step raised: its rows are taken back, so that the next plan names them again. A request whose
        cache still stands where the row began keeps it (and the pages taken for the row: the next plan needs them
        again); one whose cache the failed step had already moved on is treated like a preempted request: it keeps its
        tokens, loses its pages and is recomputed from position 0, since what the step wrote cannot be trusted and pages
        a window has passed cannot be had back. A request preempted or aborted while the plan was made stays so."""
        for row in plan.rows:
            s = row.sequence
            if s not in self._seqs:
                continue
            held = self.cache.get(s.request_id).tokens if s.request_id in self.cache else 0
            if held == row.start:
                s.computed = row.start
            else:
                self.cache.free(s.request_id)
                s.computed = 0

    def _preempt(self, v: Sequence) -> None:
        """The victim keeps every token, loses its pages and is recomputed from position 0."""
        self.cache.free(v.request_id)
        v.computed = 0
        v.preemptions += 1
        self.preemption_count += 1

    def _remove(self, s: Sequence) -> None:
        self.cache.free(s.request_id)
        self._seqs.remove(s)

    # ------------------------------------------------------------------ results
    def apply(self, plan: StepPlan, tokens: dict) -> list[TokenEvent]:
        """``tokens``: request id -> sampled token, for every row of the plan that samples. Appends the tokens,
        finishes what is done and records the cache lengths."""
        events = list(plan.aborted)
        for row in plan.rows:
            s = row.sequence
            self.cache.commit(s.request_id, row.start + row.count)
            if not row.samples:
                continue
            if s.request_id not in tokens:
                self._remove(s)
                s.finished = "error"
                events.append(TokenEvent(s.request_id, None, "error"))
                continue
            tok = int(tokens[s.request_id])
            s.tokens.append(tok)
            s.generated += 1
            reason = self._finish_reason(s, tok)
            if reason:
                s.finished = reason
                self._remove(s)
            events.append(TokenEvent(s.request_id, tok, reason))
        return events

    def _finish_reason(self, s: Sequence, tok: int) -> str | None:
        sp = s.request.sampling
        if s.generated >= sp.min_tokens:
            # ``ignore_eos`` switches off the model's stop ids (config.json's eos_token_id), not the request's own
            if tok in s.request.stop_token_ids or (not sp.ignore_eos and tok in self.options.model_stop_token_ids):
                return "stop"
        if sp.max_tokens is not None and s.generated >= sp.max_tokens:
            return "length"
        limit = self.cache.max_tokens_per_request()
        if self.options.max_context is not None:
            limit = min(limit, self.options.max_context)
        if len(s.tokens) >= limit:
            return "length"  # no room to run the token just generated and one more
        return None
