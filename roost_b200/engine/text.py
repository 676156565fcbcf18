"""Text around the token-id engine: incremental detokenisation, stop strings, the chat turn format.

The reference matches stop sequences on the host, on detokenised text, as the tokens stream in
(src/Starlings.Generation.Roost/RoostChatClient.cs:366-378): ordinal comparison, text that could be the start of a stop
sequence is held back until it is decided, the earliest match wins and among matches at the same place the longest
(src/Starlings.Roost.Generation/StopMatching.cs:36-39); the match itself is cut from the output and the request is
cancelled. No tokenizer ships with the reference or with this package: every function here takes a tokenizer object
with ``encode(str) -> ids`` (or an object with ``.ids``) and ``decode(ids) -> str``.
"""
from __future__ import annotations

from dataclasses import dataclass

REPLACEMENT = "\ufffd"   # what a decoder puts where a token sequence ends inside a character


class StopMatcher:
    """Finds the first stop string in text that arrives in pieces. ``push(piece)`` returns (text safe to emit, the stop
    string that matched or None); once a string has matched nothing more is emitted. ``flush()`` returns what was held
    back when no more text will come. The decision is the one the whole text would give, however it is cut into pieces:
    a stop string that is complete waits while another one that begins before it, or at the same place and longer, can
    still become complete."""

    def __init__(self, stop_strings=()):
        stops = [s for s in stop_strings]
        for s in stops:
            if not isinstance(s, str) or not s:
                raise ValueError("a stop string must be a non-empty string")
        self.stops = stops
        self.held = ""
        self.matched: str | None = None

    def _complete(self, text: str):
        """The earliest complete match in ``text``, the longest among those that start there: (start, stop) or None."""
        best = None
        for s in self.stops:
            at = text.find(s)
            if at >= 0 and (best is None or (at, -len(s)) < (best[0], -len(best[1]))):
                best = (at, s)
        return best

    def push(self, piece: str) -> tuple[str, str | None]:
        if self.matched is not None:
            return "", self.matched
        if not self.stops:
            return piece, None
        text = self.held + piece
        best = self._complete(text)
        # Where the earliest stop string begins that the text's end is still inside of (a proper prefix of it reaches the
        # end). Text from there on is held back; and a complete match is only final if no such string begins before it, or
        # at its start and longer: that one would win once it is complete.
        limit = len(text) if best is None else best[0] + 1
        open_at = None
        for i in range(max(0, len(text) - max(len(s) for s in self.stops) + 1), min(limit, len(text))):
            rest = len(text) - i
            if any(len(s) > rest and s.startswith(text[i:]) and (best is None or i < best[0] or len(s) > len(best[1])) for s in self.stops):
                open_at = i
                break
        if best is not None and open_at is None:
            self.matched = best[1]
            self.held = ""
            return text[: best[0]], self.matched
        if open_at is None:
            self.held = ""
            return text, None
        self.held = text[open_at:]
        return text[:open_at], None

    def flush(self) -> str:
        """No more text will come: what was held back, up to a stop string that is complete in it (``matched`` then names it)."""
        out, self.held = self.held, ""
        if self.matched is not None:
            return ""
        best = self._complete(out) if self.stops else None
        if best is not None:
            self.matched = best[1]
            return out[: best[0]]
        return out


class IncrementalDetokenizer:
    """Turns a growing list of token ids into text deltas. The whole list is decoded each time (a token may change how
    its neighbours read) and what is new beyond the text already given out is returned; a tail that ends inside a
    character (the decoder's replacement mark) waits for the tokens that complete it."""

    def __init__(self, tokenizer, **decode_options):
        self.tokenizer = tokenizer
        self.options = decode_options
        self.ids: list[int] = []
        self.given = ""

    def _decode(self) -> str:
        return self.tokenizer.decode(self.ids, **self.options)

    def push(self, token: int) -> str:
        self.ids.append(int(token))
        whole = self._decode()
        if whole.endswith(REPLACEMENT) or not whole.startswith(self.given):
            return ""
        delta, self.given = whole[len(self.given) :], whole
        return delta

    def flush(self) -> str:
        whole = self._decode()
        delta = whole[len(self.given) :] if whole.startswith(self.given) else ""
        self.given = whole
        return delta


def encode(tokenizer, text: str, **options) -> list[int]:
    ids = tokenizer.encode(text, **options)
    return list(getattr(ids, "ids", ids))


# The turn format Qwen3 checkpoints are tuned on: every message is "<|im_start|>{role}\n{content}<|im_end|>\n" and the
# prompt ends with the opening of the assistant's turn.
CHATML_TURN = "<|im_start|>{role}\n{content}<|im_end|>\n"
CHATML_REPLY = "<|im_start|>assistant\n"
CHAT_ROLES = ("system", "user", "assistant", "tool")


def render_chat(messages, turn: str = CHATML_TURN, reply: str = CHATML_REPLY) -> str:
    """The prompt text of a conversation: ``messages`` is a list of {"role": ..., "content": ...}."""
    if not messages:
        raise ValueError("a conversation needs at least one message")
    parts = []
    for i, m in enumerate(messages):
        try:
            role, content = m["role"], m["content"]
        except (KeyError, TypeError):
            raise ValueError(f"message {i} needs a 'role' and a 'content'") from None
        if role not in CHAT_ROLES:
            raise ValueError(f"message {i} has role '{role}'; expected one of {', '.join(CHAT_ROLES)}")
        if not isinstance(content, str):
            raise ValueError(f"message {i}: the content must be text")
        parts.append(turn.replace("{role}", role).replace("{content}", content))
    return "".join(parts) + reply


@dataclass
class TextUpdate:
    """A piece of generated text; the last update of a completion carries the finish reason ("stop": a stop token or a
    stop string, "length") and the usage counts, and may carry no text."""
    text: str
    finish_reason: str | None = None
    stop_string: str | None = None
    prompt_tokens: int = 0
    completion_tokens: int = 0


@dataclass
class TextCompletion:
    text: str
    finish_reason: str | None
    stop_string: str | None = None
    prompt_tokens: int = 0
    completion_tokens: int = 0
