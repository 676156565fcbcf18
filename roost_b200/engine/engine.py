"""The Python entry point: token ids in, generated token ids out.

``RoostEngine`` ties the parts together the way the reference's driver loop does
(src/Starlings.Generation.Roost/Driver/WorkerDriver.cs:325-400): admit requests, ask the scheduler for a plan,
run the plan through the step function, sample the rows that reach their last token, apply the tokens (which
finishes requests and frees their pages), repeat. Its surface follows the reference's client
(src/Starlings.Generation.Roost/RoostChatClient.cs:206-231,301-451): a raw completion over prompt token ids with
options ``max_output_tokens``, ``temperature`` (unset means greedy, as the reference's chat API treats it,
ChatRequestBuilder.cs:180), ``top_p``, ``top_k``, ``min_p``, ``seed``, ``stop_token_ids``; updates carry the
new token, the last one a finish reason ("stop" or "length") and the usage counts. The reference ships no
tokenizer in its repository, so token ids are the contract here; text goes in and out only when the caller
passes a tokenizer object with ``encode`` and ``decode``.
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Iterator

import torch

from ..sampling.sampler import Sampler, SamplingRow
from .executor import StepEntry, StepExecutor
from .model import Model, load_model
from .request import GREEDY, Request, RequestError, SamplingParameters, TokenEvent
from .scheduler import Scheduler, SchedulerOptions, StepPlan
from .text import (IncrementalDetokenizer, StopMatcher, TextCompletion, TextUpdate, encode, render_chat)


class _Done:
    def synchronize(self) -> None:
        pass


@dataclass
class _InFlight:
    """A decode step that was started before the tokens of the step before it were read (see ``RoostEngine.step``)."""
    prep: object                  # the executor's PreparedDecode
    ids_device: torch.Tensor      # the tokens it samples, on the device
    ids_host: torch.Tensor        # their pinned copy (followed by the kernels' status words), valid once ``event`` has passed
    event: object
    fed: list | None = None       # the tokens it was fed, once the host has read them


@dataclass
class GenerationOptions:
    """Options of one completion, with the reference's names in snake case."""
    max_output_tokens: int | None = None
    temperature: float | None = None       # None or 0: greedy
    top_p: float | None = None
    top_k: int | None = None
    min_p: float | None = None
    seed: int | None = None
    stop_token_ids: tuple = ()
    ignore_eos: bool = False               # generate past the model's stop ids (stop_token_ids above still end the request)
    repetition_penalty: float | None = None   # None or 1: off
    frequency_penalty: float | None = None    # None or 0: off
    presence_penalty: float | None = None
    logprobs: bool = False                     # the logprob of every generated token
    top_logprobs: int = 0                      # and of this many most likely alternatives (needs logprobs)
    allowed_token_ids: tuple | None = None     # the only tokens that may be generated; None: all

    def sampling(self) -> SamplingParameters:
        return SamplingParameters(temperature=self.temperature or 0.0, top_p=1.0 if self.top_p is None else self.top_p,
                                  top_k=0 if self.top_k in (None, -1) else self.top_k, min_p=self.min_p or 0.0, seed=self.seed,
                                  max_tokens=self.max_output_tokens, ignore_eos=self.ignore_eos,
                                  repetition_penalty=1.0 if self.repetition_penalty is None else self.repetition_penalty,
                                  frequency_penalty=self.frequency_penalty or 0.0, presence_penalty=self.presence_penalty or 0.0,
                                  logprobs=self.logprobs, top_logprobs=self.top_logprobs,
                                  allowed_token_ids=None if self.allowed_token_ids is None else tuple(self.allowed_token_ids))


@dataclass
class CompletionUpdate:
    request_id: object
    token: int | None
    finish_reason: str | None = None
    prompt_tokens: int = 0
    completion_tokens: int = 0
    logprob: float | None = None
    top_logprobs: list | None = None


@dataclass
class Completion:
    request_id: object
    token_ids: list = field(default_factory=list)
    finish_reason: str | None = None
    prompt_tokens: int = 0
    logprobs: list | None = None         # one a token, when asked for
    top_logprobs: list | None = None     # [(token id, logprob)] lists, one a token, when asked for


class RoostEngine:
    def __init__(self, model, *, dtype: str | torch.dtype = "bfloat16", device: str = "cuda", page_size: int = 16,
                 attention_blocks: int | None = None, kv_fraction: float = 0.9, max_sequences: int = 64, max_tokens: int = 2048,
                 max_chunk_tokens: int | None = None, seed: int | None = None, chain_steps: bool = True):
        """``model``: a folder with config.json and model.safetensors, or a built ``Model``. ``attention_blocks``:
        pages in each paged pool (else ``kv_fraction`` of the free device memory); ``max_tokens`` and
        ``max_sequences``: the largest token and row count of a step (the reference's worker flags of the same
        names, src/Starlings.Roost.WorkerHost/WorkerArguments.cs:51-58). ``chain_steps``: while every live request
        decodes, the next step is started on the device before this step's tokens have been read (the reference's
        planner keeps plans in flight while it makes later ones, ``_inFlight``,
        src/Starlings.Roost.Engine/Scheduling/StepPlanner.cs:102,345,951; it does not start a step on tokens the host has
        not seen, which is this engine's own addition); the tokens are the same with it and without."""
        if isinstance(dtype, str):
            dtype = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}[dtype]
        self.model: Model = model if isinstance(model, Model) else load_model(model, dtype, device)
        self.executor = StepExecutor(self.model, page_size=page_size, num_pages=attention_blocks, max_requests=max_sequences,
                                     kv_fraction=kv_fraction)
        spec = self.model.spec
        self.scheduler = Scheduler(self.executor.cache, SchedulerOptions(
            max_tokens_per_step=max_tokens, max_sequences_per_step=max_sequences, max_chunk_tokens=max_chunk_tokens,
            model_stop_token_ids=tuple(spec.stop_token_ids), max_context=spec.max_positions or None))
        self.sampler = Sampler(self.model.rt.kernels, self.model.rt.device, max_requests=max_sequences)
        self._extras: dict = {}     # request id -> (logprob, alternatives) of the token this step sampled
        self._seed_source = random.Random(seed)
        self._seeds: dict = {}
        self._next_id = 0
        self.steps = 0
        self.last_plan: StepPlan | None = None
        self._prepared = None     # the next decode step's tables, made while the device ran the last one
        self._inflight: _InFlight | None = None   # the next decode step, already running
        self.chain_steps = chain_steps
        self._status_with_tokens = hasattr(self.model.rt.kernels, "status_snapshot") and self.model.rt.device.type == "cuda"
        self.chained_steps = 0    # steps that were running before the tokens of the step before them had been read

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_token_ids, sampling: SamplingParameters = GREEDY, *, request_id=None, stop_token_ids=(),
                    priority: int = 0, deadline: float | None = None):
        if request_id is None:
            request_id = f"req-{self._next_id}"
            self._next_id += 1
        vocab = self.model.spec.vocab
        for t in prompt_token_ids:
            if not 0 <= int(t) < vocab:
                raise RequestError("InvalidOption", f"prompt token id {t} is outside the vocabulary of {vocab}")
        if sampling.allowed_token_ids is not None and any(int(t) >= vocab for t in sampling.allowed_token_ids):
            raise RequestError("InvalidOption", f"an allowed token id is outside the vocabulary of {vocab}")
        req = Request(request_id, [int(t) for t in prompt_token_ids], sampling, tuple(stop_token_ids), priority, deadline)
        self.scheduler.add(req)
        # a request without a seed gets an engine-chosen one (src/Starlings.Generation.Roost/RoostChatClient.cs:329)
        self._seeds[request_id] = sampling.seed if sampling.seed is not None else self._seed_source.getrandbits(64)
        return request_id

    def cancel(self, request_id) -> bool:
        self._seeds.pop(request_id, None)
        self._release(request_id)
        return self.scheduler.cancel(request_id)

    def _release(self, request_id) -> None:
        release = getattr(self.sampler, "release", None)
        if release is not None:
            release(request_id)

    def has_unfinished(self) -> bool:
        return self.scheduler.unfinished > 0

    # ------------------------------------------------------------------ one engine step
    def step(self) -> list[TokenEvent]:
        """Plans, runs and applies one step; returns the tokens it produced (possibly none: a step of prompt
        portions that reach no request's last token)."""
        plan = self.scheduler.plan()
        self.last_plan = plan
        if plan is None:
            return []
        tokens = {}
        if plan.rows:
            try:
                tokens = self._run(plan)
            except Exception:
                # nothing of this plan is applied: its rows are planned again from where the cache stands, a step that
                # was started ahead is dropped, and the error goes to the caller with the engine still usable
                self._prepared = self._inflight = None
                self.scheduler.rollback(plan)
                raise
        events = self.scheduler.apply(plan, tokens)
        for e in events:
            extra = self._extras.pop(e.request_id, None) if self._extras else None
            if extra is not None and e.token is not None:
                e.logprob, e.top_logprobs = extra
            if e.finish_reason is not None:
                self._seeds.pop(e.request_id, None)
                self._release(e.request_id)
        return events

    def _run(self, plan: StepPlan) -> dict:
        """Runs the plan's rows through the step function and the sampler; request id -> sampled token."""
        tokens = {}
        entries = [StepEntry(r.sequence.request_id, r.tokens, [r.count - 1] if r.samples else [], r.start) for r in plan.rows]
        prepared, self._prepared = self._prepared, None
        inflight, self._inflight = self._inflight, None
        sampling_rows = [r for r in plan.rows if r.samples]
        ids_device = ids_host = event = extras_host = None
        keep = None
        if inflight is not None and len(sampling_rows) == len(plan.rows):
            keep = self.executor.adoptable(inflight.prep, entries)
            if keep is not None and any(e.tokens[0] != inflight.fed[i] for e, i in zip(entries, keep)):
                keep = None    # the step was fed other tokens than the plan names: it does not stand
        if keep is not None:
            # this step is running already (or done): it was started with the tokens on the device
            self.executor.adopt_prepared(inflight.prep, keep)
            self.chained_steps += 1
            ids_device, ids_host, event = inflight.ids_device, inflight.ids_host, inflight.event
            if len(keep) != ids_device.numel():
                ids_device = ids_device[torch.tensor(keep, dtype=torch.long).to(ids_device.device, non_blocking=True)]
        else:
            # (a step in flight that does not stand is dropped: what it wrote lies beyond its requests' committed
            # lengths and is written again, and the pages it took stay with their requests)
            if prepared is not None and self.executor.matches_prepared(prepared, entries):
                logits = self.executor.run_prepared(prepared, entries)
            else:
                logits = self.executor.step(entries)
            if sampling_rows:
                ids_device = self.sampler(logits, [self._sampling_row(r, 0) for r in sampling_rows])
                extras_host = self._extras_to_host()
                ids_host, event = self._to_host(ids_device)
                keep = list(range(len(sampling_rows)))
        if sampling_rows:
            # While the device runs this step: the next one, should it be these rows' next tokens and nothing else
            # (no request waiting for its prompt). Its tables are made now; with ``chain_steps`` it is also started
            # now, fed with this step's tokens on the device, and the host reads this step's tokens meanwhile.
            if len(sampling_rows) == len(plan.rows) and all(r.count == 1 for r in plan.rows) and self._decode_only():
                prep = self.executor.prepare_decode([r.sequence.request_id for r in plan.rows])
                # (a request with penalties or logprobs is sampled from its accepted tokens and hands back more than an
                # id: its steps are not started ahead)
                plain_rows = not any(r.sequence.request.sampling.penalised or r.sequence.request.sampling.logprobs for r in plan.rows)
                if prep is not None and self.chain_steps and plain_rows:
                    nxt = self.executor.launch_prepared(prep, ids_device)
                    nxt_ids = self.sampler(nxt, [self._sampling_row(r, 1) for r in plan.rows])
                    self._inflight = _InFlight(prep, nxt_ids, *self._to_host(nxt_ids))
                else:
                    self._prepared = prep
            event.synchronize()
            host = ids_host.tolist()
            if any(host[-4:-1]):
                self.check_device()   # a kernel gave up a bounded wait: this step's tokens are not valid (raises)
            ids = [host[i] for i in keep]
            if self._inflight is not None:
                self._inflight.fed = ids
            tokens = {r.sequence.request_id: t for r, t in zip(sampling_rows, ids)}
            if extras_host is not None:
                self._extras = self._read_extras(extras_host, sampling_rows)
        self.steps += 1
        if not self._status_with_tokens and self.steps % self.STATUS_EVERY == 0:
            self.check_device()
        return tokens

    def _sampling_row(self, r, ahead: int) -> SamplingRow:
        """The sampler's view of a planned row; ``ahead``: tokens of the request that are sampled but not yet accepted."""
        s = r.sequence
        p = s.request.sampling
        if p.penalised:
            return SamplingRow(p, self._seeds[s.request_id], s.generated + ahead, s.request_id, s.tokens[: s.prompt_len],
                               s.tokens[s.prompt_len : s.prompt_len + s.generated])
        return SamplingRow(p, self._seeds[s.request_id], s.generated + ahead)

    def _extras_to_host(self):
        """Starts the copies of what the last sampling call computed beside the ids; None when no row asked."""
        ex = getattr(self.sampler, "extras", None)     # (a caller may have put a plain function in the sampler's place)
        if ex is None or ex.logprobs is None:
            return None
        pin = ex.logprobs.device.type == "cuda"
        out = []
        for t in (ex.logprobs, ex.top_ids, ex.top_logprobs):
            if t is None:
                out.append(None)
                continue
            host = torch.empty(t.shape, dtype=t.dtype, pin_memory=pin)
            host.copy_(t, non_blocking=True)
            out.append(host)
        return out

    @staticmethod
    def _read_extras(extras_host, sampling_rows) -> dict:
        lp, top_ids, top_vals = extras_host
        lp = lp.tolist()
        out = {}
        for i, r in enumerate(sampling_rows):
            p = r.sequence.request.sampling
            if not p.logprobs:
                continue
            alternatives = None
            if p.top_logprobs and top_ids is not None:
                alternatives = list(zip(top_ids[i, : p.top_logprobs].tolist(), top_vals[i, : p.top_logprobs].tolist()))
            out[r.sequence.request_id] = (lp[i], alternatives)
        return out

    STATUS_EVERY = 256   # steps between looks at the kernels' status words when no step reads them with its tokens

    def _to_host(self, ids_device: torch.Tensor):
        """Starts the copy of sampled ids to pinned host memory; (the host tensor, the event that says it has arrived).
        The host tensor ends in four more words: the kernels' error words as they stand after this step's kernels (0: no
        bounded wait was given up) and a 1, written by the device in stream order, so that the wait for the tokens is
        also the look at the status and no generation returns tokens of a step whose kernels gave up."""
        n = ids_device.numel()
        if ids_device.device.type != "cuda":
            return torch.cat([ids_device.reshape(-1).to(torch.int32), torch.tensor([0, 0, 0, 1], dtype=torch.int32)]), _Done()
        host = torch.zeros(n + 4, dtype=ids_device.dtype, pin_memory=True)
        host[:n].copy_(ids_device.reshape(-1), non_blocking=True)
        if self._status_with_tokens:
            self.model.rt.kernels.status_snapshot(host[n:])
        event = torch.cuda.Event()
        event.record()
        return host, event

    def check_device(self) -> None:
        """Raises if a kernel gave up one of its bounded waits since the last look (its results were then not valid)."""
        check = getattr(self.model.rt.kernels, "check_device_status", None)
        if check is not None:
            check()

    def _decode_only(self) -> bool:
        """Every live request has its prompt in the cache: the next step can only be one more token for each."""
        return all(s.computed >= s.prompt_len and s.request_id in self.executor.cache for s in self.scheduler.sequences())

    # ------------------------------------------------------------------ completions
    def generate(self, prompts: list, options: GenerationOptions | list | None = None) -> list[Completion]:
        """Runs every prompt (a list of token ids each) to its end; results in the order of the prompts."""
        if options is None:
            options = GenerationOptions()
        opts = options if isinstance(options, list) else [options] * len(prompts)
        results = {}
        order = []
        for prompt, o in zip(prompts, opts):
            rid = self.add_request(prompt, o.sampling(), stop_token_ids=o.stop_token_ids)
            results[rid] = Completion(rid, [], None, len(prompt))
            order.append(rid)
        while any(results[r].finish_reason is None for r in order):
            if not self.has_unfinished():
                break
            for e in self.step():
                if e.request_id in results:
                    if e.token is not None:
                        results[e.request_id].token_ids.append(e.token)
                        if e.logprob is not None:
                            c = results[e.request_id]
                            c.logprobs = (c.logprobs or []) + [e.logprob]
                            if e.top_logprobs is not None:
                                c.top_logprobs = (c.top_logprobs or []) + [e.top_logprobs]
                    if e.finish_reason is not None:
                        results[e.request_id].finish_reason = e.finish_reason
        return [results[r] for r in order]

    def stream_completion(self, prompt_token_ids, options: GenerationOptions | None = None) -> Iterator[CompletionUpdate]:
        """One request, one update per generated token; the last update carries the finish reason and usage.
        Other live requests keep running in the same steps."""
        o = options or GenerationOptions()
        rid = self.add_request(prompt_token_ids, o.sampling(), stop_token_ids=o.stop_token_ids)
        produced = 0
        done = False
        try:
            while not done:
                if not self.has_unfinished():
                    break
                for e in self.step():
                    if e.request_id != rid:
                        continue
                    if e.token is not None:
                        produced += 1
                    done = e.finish_reason is not None
                    yield CompletionUpdate(rid, e.token, e.finish_reason, len(prompt_token_ids), produced, e.logprob, e.top_logprobs)
        finally:
            if not done:
                self.cancel(rid)   # the caller stopped listening (a stop string matched, say): out of the next step

    # ------------------------------------------------------------------ text in, text out (the caller brings the tokenizer)
    def stream_text(self, tokenizer, prompt: str, options: GenerationOptions | None = None, stop=(),
                    encode_options: dict | None = None, decode_options: dict | None = None) -> Iterator[TextUpdate]:
        """A raw completion (no chat template) as text deltas, with stop strings: they are matched on the detokenised
        text on the host as the tokens arrive, text that could be the start of one is held back until it is decided,
        the match is cut from the output, the request is cancelled and the completion ends with "stop"
        (src/Starlings.Generation.Roost/RoostChatClient.cs:366-378). The last update carries the finish reason and the
        usage counts. ``tokenizer``: ``encode(str) -> ids`` (or an object with ``.ids``) and ``decode(ids) -> str``."""
        matcher = StopMatcher(stop)
        ids = encode(tokenizer, prompt, **(encode_options or {}))
        if not ids:
            raise RequestError("InvalidOption", "the prompt has no tokens")
        detok = IncrementalDetokenizer(tokenizer, **(decode_options or {}))
        o = options or GenerationOptions()
        rid = self.add_request(ids, o.sampling(), stop_token_ids=o.stop_token_ids)
        produced, reason, live = 0, None, True
        try:
            while reason is None:
                if not self.has_unfinished():
                    break
                for e in self.step():
                    if e.request_id != rid:
                        continue
                    stop_token = e.finish_reason == "stop"
                    if e.token is not None:
                        produced += 1
                        # a stop token ends the text: it is not part of it
                        emit, matched = matcher.push("" if stop_token else detok.push(e.token))
                        if matched is not None:
                            if emit:
                                yield TextUpdate(emit)
                            reason = "stop"
                            live = e.finish_reason is None
                            break
                        if emit:
                            yield TextUpdate(emit)
                    if e.finish_reason is not None:
                        live = False
                        if not stop_token:
                            tail, _ = matcher.push(detok.flush())
                            tail += matcher.flush()     # (a stop string that waited for a longer one is decided here)
                            if tail:
                                yield TextUpdate(tail)
                            reason = "stop" if matcher.matched is not None else e.finish_reason
                        else:
                            tail = matcher.flush()
                            if tail:
                                yield TextUpdate(tail)
                            reason = "stop"
                        break
        finally:
            if live:
                self.cancel(rid)     # stopped on a string, or abandoned by the caller: out of the next step
        yield TextUpdate("", reason, matcher.matched, len(ids), produced)

    def complete_text(self, tokenizer, prompt: str, options: GenerationOptions | None = None, stop=(), **kw) -> TextCompletion:
        """Text in, text out; see ``stream_text``. The result's ``text`` excludes a matched stop string."""
        text, last = [], None
        for u in self.stream_text(tokenizer, prompt, options, stop, **kw):
            text.append(u.text)
            last = u
        return TextCompletion("".join(text), last.finish_reason, last.stop_string, last.prompt_tokens, last.completion_tokens)

    def stream_chat(self, tokenizer, messages, options: GenerationOptions | None = None, stop=(), turn: str | None = None,
                    reply: str | None = None, **kw) -> Iterator[TextUpdate]:
        """The reply to a conversation (a list of {"role", "content"}) as text deltas: the messages are rendered in the
        turn format the Qwen3 checkpoints are tuned on (``text.render_chat``; ``turn`` and ``reply`` give another) and
        completed like ``stream_text``; the end-of-turn mark is a stop string unless the caller names its own."""
        from .text import CHATML_REPLY, CHATML_TURN
        prompt = render_chat(messages, turn or CHATML_TURN, reply if reply is not None else CHATML_REPLY)
        return self.stream_text(tokenizer, prompt, options, tuple(stop) or ("<|im_end|>",), **kw)

    def chat(self, tokenizer, messages, options: GenerationOptions | None = None, stop=(), **kw) -> TextCompletion:
        """The assistant's reply to ``messages`` as one text; see ``stream_chat``."""
        text, last = [], None
        for u in self.stream_chat(tokenizer, messages, options, stop, **kw):
            text.append(u.text)
            last = u
        return TextCompletion("".join(text), last.finish_reason, last.stop_string, last.prompt_tokens, last.completion_tokens)

    # ------------------------------------------------------------------ figures
    def stats(self) -> dict:
        return {"steps": self.steps, "kv_cache_usage": self.executor.cache.usage(), "preemptions": self.scheduler.preemption_count,
                "kernel_launches": self.model.rt.kernels.launches}
