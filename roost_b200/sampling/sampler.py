"""Sampling above the step function: greedy, or temperature with top-k, top-p and min-p, on the device; before the
draw the reference's repetition, frequency and presence penalties, after it the token's logprob and the most likely
alternatives.

One call samples every row of a step that wants a token. A batch of greedy rows goes to the argmax kernel;
otherwise the per-row parameter tables are uploaded in one copy and the sampling kernel runs (greedy rows in
such a batch are rows with temperature 0). The draw of a row depends on its own seed and on how many tokens
its request has generated (the Philox offset), not on the batch or the row index, so a request that is
preempted and recomputed draws the same tokens again
(src/Starlings.Roost.Engine/Scheduling/StepPlanner.cs:955-968, src/Starlings.Roost.Ops/CpuOps.Sampling.cs:39-41).

Penalties (src/Starlings.Roost.Ops/CpuOps.Sampling.cs:13-17,195-237) need, per request, how often each token was
generated and which tokens its prompt holds. Both live on the device, one slot a request that asked for penalties: a
row of int32 counts over the vocabulary and a row of bits. A third row of bits is the request's token mask (:18-19): the
tokens it allows; the others are removed after the penalties. They are brought up to date from the request's accepted
tokens at the start of every call (usually one token), so a step that is rolled back or a request that is preempted and
recomputed counts nothing twice. Logprobs (:166-176,516-603) are the log-softmax of the raw logits, before penalties and
temperature.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..engine.request import SamplingParameters

_MASK64 = (1 << 64) - 1


@dataclass
class SamplingRow:
    params: SamplingParameters
    seed: int          # 64-bit, already chosen for requests that gave none
    offset: int        # tokens the request has generated so far
    request_id: object = None      # needed (with the two lists) by rows that ask for penalties
    prompt: list | None = None     # the request's prompt tokens
    output: list | None = None     # the tokens it has generated and the engine has accepted, in order


@dataclass
class SampleExtras:
    """What a call computed beside the ids, on the device: None where no row asked."""
    logprobs: torch.Tensor | None = None      # float32 [S]
    top_ids: torch.Tensor | None = None       # int32 [S, K]
    top_logprobs: torch.Tensor | None = None  # float32 [S, K]


class Sampler:
    def __init__(self, kernels, device, max_requests: int = 64):
        self.kernels = kernels
        self.device = torch.device(device)
        self.max_requests = max_requests
        self._workspace: torch.Tensor | None = None
        self._counts: torch.Tensor | None = None      # int32 [max_requests, vocab]
        self._bits: torch.Tensor | None = None        # int32 [max_requests, (vocab + 31) // 32]: the prompts' tokens
        self._mask: torch.Tensor | None = None        # the same shape: the tokens a request allows (all ones: every token)
        self._slots: dict = {}                        # request id -> [slot, output tokens counted so far]
        self._free: list[int] = []
        self.extras = SampleExtras()                  # of the last call

    # ------------------------------------------------------------------ penalty state
    def release(self, request_id) -> None:
        """The request is over: its slot of counts serves the next one."""
        entry = self._slots.pop(request_id, None)
        if entry is not None:
            self._free.append(entry[0])

    def _grow(self) -> None:
        """Twice as many slots. A request keeps its slot from its first sampled token to its end, also while it waits
        (preempted, or behind requests that came later but are ordered before it), so more requests than a step has rows
        can hold one."""
        old = self.max_requests
        pad = lambda t, fill: torch.cat([t, torch.full_like(t, fill)])
        self._counts, self._bits, self._mask = pad(self._counts, 0), pad(self._bits, 0), pad(self._mask, -1)
        self.max_requests = 2 * old
        self._free = list(range(2 * old - 1, old - 1, -1))

    def _to_device(self, values, dtype) -> torch.Tensor:
        host = torch.tensor(values, dtype=dtype)
        if self.device.type == "cuda":
            host = host.pin_memory()
        return host.to(self.device, non_blocking=True)

    def _penalty_slots(self, rows: list[SamplingRow], vocab: int) -> list[int]:
        """The slot of every row (-1: no penalties), with the counts brought up to date with the rows' accepted tokens."""
        if self._counts is None or self._counts.shape[1] != vocab:
            self._counts = torch.zeros((self.max_requests, vocab), dtype=torch.int32, device=self.device)
            self._bits = torch.zeros((self.max_requests, (vocab + 31) // 32), dtype=torch.int32, device=self.device)
            self._mask = torch.full((self.max_requests, (vocab + 31) // 32), -1, dtype=torch.int32, device=self.device)
            self._slots.clear()
            self._free = list(range(self.max_requests - 1, -1, -1))
        slots, new_slots, new_ids = [], [], []
        for r in rows:
            if not r.params.penalised:
                slots.append(-1)
                continue
            if r.request_id is None or r.prompt is None or r.output is None:
                raise ValueError("a row with penalties needs its request's id, prompt and output tokens")
            entry = self._slots.get(r.request_id)
            if entry is None:
                if not self._free:
                    self._grow()
                entry = self._slots[r.request_id] = [self._free.pop(), 0]
                self._counts[entry[0]].zero_()
                self._bits[entry[0]].zero_()
                if r.prompt:
                    self.kernels.sample_prompt_bits(self._bits[entry[0]], self._to_device(r.prompt, torch.int32))
                if r.params.allowed_token_ids is not None:
                    if max(r.params.allowed_token_ids) >= vocab:
                        raise ValueError(f"allowed token id {max(r.params.allowed_token_ids)} is outside the vocabulary of {vocab}")
                    self._mask[entry[0]].zero_()
                    self.kernels.sample_prompt_bits(self._mask[entry[0]], self._to_device(list(r.params.allowed_token_ids), torch.int32))
                else:
                    self._mask[entry[0]].fill_(-1)
            slot, counted = entry
            if counted > len(r.output):      # cannot be: accepted tokens are never taken back
                raise RuntimeError("a request's output shrank under its penalty counts")
            new_ids += r.output[counted:]
            new_slots += [slot] * (len(r.output) - counted)
            entry[1] = len(r.output)
            slots.append(slot)
        if new_ids:
            self.kernels.sample_count_tokens(self._counts, self._to_device(new_slots, torch.int32), self._to_device(new_ids, torch.int32))
        return slots

    # ------------------------------------------------------------------ a step's rows
    def __call__(self, logits: torch.Tensor, rows: list[SamplingRow]) -> torch.Tensor:
        """logits [S, vocab] float32 on the device; returns int32 token ids [S] on the device. ``self.extras`` then
        holds the logprobs of the rows that asked for them."""
        if logits.shape[0] != len(rows):
            raise ValueError(f"{logits.shape[0]} rows of logits for {len(rows)} sampling rows")
        self.extras = SampleExtras()
        S, V = logits.shape
        raw = logits
        if any(r.params.penalised for r in rows):
            slots = self._penalty_slots(rows, V)
            table = np.empty(4 * S, np.int32)
            table[0:S] = slots
            table[S : 2 * S] = np.asarray([r.params.repetition_penalty for r in rows], np.float32).view(np.int32)
            table[2 * S : 3 * S] = np.asarray([r.params.presence_penalty for r in rows], np.float32).view(np.int32)
            table[3 * S : 4 * S] = np.asarray([r.params.frequency_penalty for r in rows], np.float32).view(np.int32)
            dev = self._to_device(table, torch.int32)
            logits = self.kernels.sample_penalise(logits, self._counts, self._bits, dev[0:S], dev[S : 2 * S].view(torch.float32),
                                                  dev[2 * S : 3 * S].view(torch.float32), dev[3 * S : 4 * S].view(torch.float32), self._mask)
        ids = self._draw(logits, rows)
        if any(r.params.logprobs for r in rows):
            top = max(r.params.top_logprobs for r in rows)
            lp, top_ids, top_vals = self.kernels.sample_logprobs(raw, ids, top)
            self.extras = SampleExtras(lp, top_ids if top else None, top_vals if top else None)
        return ids

    def _draw(self, logits: torch.Tensor, rows: list[SamplingRow]) -> torch.Tensor:
        if all(r.params.greedy for r in rows):
            return self.kernels.argmax(logits)
        S, V = logits.shape
        # one pinned buffer: temperature, top_k, top_p, min_p as 32-bit words, then seeds and offsets as 64-bit
        host = torch.empty(4 * S + 4 * S, dtype=torch.int32, pin_memory=self.device.type == "cuda")
        hv = host.numpy()
        hv[0:S] = np.asarray([r.params.temperature for r in rows], np.float32).view(np.int32)
        hv[S : 2 * S] = np.asarray([max(r.params.top_k, 0) for r in rows], np.int32)
        hv[2 * S : 3 * S] = np.asarray([r.params.top_p for r in rows], np.float32).view(np.int32)
        hv[3 * S : 4 * S] = np.asarray([r.params.min_p for r in rows], np.float32).view(np.int32)
        hv[4 * S : 6 * S] = np.asarray([r.seed & _MASK64 for r in rows], np.uint64).view(np.int32)
        hv[6 * S : 8 * S] = np.asarray([r.offset & _MASK64 for r in rows], np.uint64).view(np.int32)
        dev = host.to(self.device, non_blocking=True)
        if self._workspace is None or self._workspace.shape[0] < S or self._workspace.shape[1] != V:
            self._workspace = torch.empty((S, V), dtype=torch.float32, device=self.device)
        return self.kernels.sample(logits, dev[0:S].view(torch.float32), dev[S : 2 * S], dev[2 * S : 3 * S].view(torch.float32),
                                   dev[3 * S : 4 * S].view(torch.float32), dev[4 * S : 6 * S].view(torch.int64),
                                   dev[6 * S : 8 * S].view(torch.int64), self._workspace[:S])
