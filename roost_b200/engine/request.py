"""Requests as the engine sees them: token ids in, sampling parameters, limits.

Field names and defaults are the reference's request contract
(src/Starlings.Roost.Abstractions/Requests/Request.cs:19-68 for the sampling parameters, :148-200 for the
request): temperature 1 unless set (0 means greedy), top_p 1 disables, top_k 0 disables, min_p 0 disables, a
missing seed is replaced by an engine-chosen one, stop token ids are the model's plus the request's; repetition
penalty 1 and frequency and presence penalties 0 disable (the ranges are the chat builder's,
src/Starlings.Generation.Roost/ChatRequestBuilder.cs:199-223,240-245); logprobs off, at most 20 alternatives a token.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field


class RequestError(ValueError):
    """A request the engine refuses at admission; ``kind`` is the reference's refusal name."""

    def __init__(self, kind: str, message: str):
        super().__init__(f"{kind}: {message}")
        self.kind = kind


@dataclass(frozen=True)
class SamplingParameters:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    seed: int | None = None
    max_tokens: int | None = None
    min_tokens: int = 0
    ignore_eos: bool = False                  # the model's stop ids do not end the request (its own stop_token_ids still do)
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    logprobs: bool = False
    top_logprobs: int = 0
    allowed_token_ids: tuple | None = None    # the only tokens that may be generated (the reference's token mask); None: all

    MAX_TOP_LOGPROBS = 20

    def validate(self) -> None:
        if self.temperature < 0:
            raise RequestError("InvalidOption", f"temperature {self.temperature} is negative")
        if not 0 < self.top_p <= 1:
            raise RequestError("InvalidOption", f"top_p {self.top_p} is outside (0, 1]")
        if self.top_k < -1:
            raise RequestError("InvalidOption", f"top_k {self.top_k} is below -1")
        if not 0 <= self.min_p <= 1:
            raise RequestError("InvalidOption", f"min_p {self.min_p} is outside [0, 1]")
        if self.max_tokens is not None and self.max_tokens <= 0:
            raise RequestError("InvalidOption", f"max_tokens {self.max_tokens} must be positive")
        if not (math.isfinite(self.repetition_penalty) and self.repetition_penalty > 0):
            raise RequestError("InvalidOption", f"repetition_penalty must be a positive number; got {self.repetition_penalty}")
        for name in ("frequency_penalty", "presence_penalty"):
            v = getattr(self, name)
            if not (math.isfinite(v) and -2 <= v <= 2):
                raise RequestError("InvalidOption", f"{name} must be in [-2, 2]; got {v}")
        if not 0 <= self.top_logprobs <= self.MAX_TOP_LOGPROBS:
            raise RequestError("InvalidOption", f"top_logprobs must be in [0, {self.MAX_TOP_LOGPROBS}]; got {self.top_logprobs}")
        if self.top_logprobs > 0 and not self.logprobs:
            raise RequestError("InvalidOption", "top_logprobs needs logprobs set to true")
        if self.allowed_token_ids is not None and (not self.allowed_token_ids or any(int(t) < 0 for t in self.allowed_token_ids)):
            raise RequestError("InvalidOption", "allowed_token_ids must name at least one token and no negative id")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0

    @property
    def penalised(self) -> bool:
        """The request's logits are changed before the draw (penalties, or tokens removed): it has a slot of sampler state."""
        return (self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0 or self.presence_penalty != 0.0
                or self.allowed_token_ids is not None)


GREEDY = SamplingParameters(temperature=0.0)


@dataclass
class Request:
    request_id: object
    prompt_token_ids: list
    sampling: SamplingParameters = field(default_factory=SamplingParameters)
    stop_token_ids: tuple = ()
    priority: int = 0                 # higher runs first
    deadline: float | None = None     # earlier runs first among equal priorities; None last


@dataclass
class TokenEvent:
    """One generated token of one request; ``finish_reason`` is set on the request's last token
    ("stop": a stop token, "length": max_tokens or the context's end) or, with ``token`` None, when the request
    was aborted ("aborted": it can never fit in the cache)."""
    request_id: object
    token: int | None
    finish_reason: str | None = None
    logprob: float | None = None          # of the token, when the request asked for logprobs
    top_logprobs: list | None = None      # [(token id, logprob)] of the highest raw logits, when it asked for alternatives
