"""Interfaces of the parts a model is assembled from, and the registries that map a spec's ``kind`` to a class.

A part is built from its spec and a ``Runtime`` (compute dtype, device, kernel library), declares the
parameters it wants by local name and shape, receives them through ``load`` and is then called with
tensors. No part knows which model it is in, which layer it is, or what its neighbours are: the spec carries
every size and constant. The reference expresses the same rule as op arguments on a node list
(src/Starlings.Roost.Models.Tiny/RoostTiny.cs:39-56) and checks at load that every op has a kernel
(src/Starlings.Roost.ModelCompiler/Emit/Emitter.cs:315-334); here a part's constructor refuses sizes no
kernel serves.

Adding a part: subclass the interface below, give the spec class a new ``kind`` and call the matching
``register_*`` function (a test does this with a toy mixer without touching this package).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable

import torch


@dataclass(frozen=True)
class ParamDecl:
    """A parameter a part wants. ``row_splits``: when the checkpoint stores the parameter as several
    tensors concatenated along dimension 0, their row counts in order."""
    shape: tuple
    row_splits: tuple | None = None
    # "matrix": converted to the compute dtype; "vector": kept in its stored dtype (32-bit stays 32-bit) in the
    # bfloat16 path; "table": integer tables become int32. In the 32-bit path every float becomes float32.
    role: str = "matrix"


@dataclass(frozen=True)
class CacheNeed:
    """What one run of a mixer keeps between steps. ``paged``: ``planes`` tensors of ``kv_heads`` x ``head_dim`` per
    token (2: keys and values; 1: one vector a token, a latent from which a mixer makes both), every earlier token
    (window None) or the last ``window`` tokens. ``state``: one tensor of ``state_shape`` per live request, zeroed when
    the request's first token arrives."""
    kind: str                       # "paged" | "state"
    kv_heads: int = 0
    head_dim: int = 0
    window: int | None = None
    planes: int = 2
    state_shape: tuple = ()
    state_dtype: torch.dtype = torch.float32


class Runtime:
    """What every part is built with: the compute dtype of activations (and of the cache), the device, and
    the kernel library handle (None only for declaring parameters on a machine without a GPU)."""

    def __init__(self, dtype: torch.dtype, device, kernels=None):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype {dtype} is not float32 or bfloat16")
        self.dtype = dtype
        self.device = torch.device(device)
        self.kernels = kernels
        # products of at most 64 rows: "auto" | "library" | "stream" (parts/linear.py)
        self.small_gemm = os.environ.get("ROOST_SMALL_GEMM", "auto")
        if self.small_gemm not in ("auto", "library", "stream", "split"):
            raise ValueError(f"ROOST_SMALL_GEMM={self.small_gemm!r} is not one of auto, library, stream, split")

    @property
    def full_precision(self) -> bool:
        return self.dtype == torch.float32


class Part:
    spec = None
    # False for a part whose call reads device values on the host or launches a number of kernels that depends on the
    # data (routing written in Python, say): a model with such a part runs its steps eagerly instead of
    # replaying captured CUDA graphs. A class that does not derive from Part may set the attribute all the same.
    capturable = True

    @classmethod
    def parameters(cls, spec) -> dict[str, ParamDecl]:
        return {}

    def load(self, params: dict[str, torch.Tensor]) -> None:
        if params:
            raise ValueError(f"{type(self).__name__} takes no parameters")


class Norm(Part):
    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_norm(self, x: torch.Tensor, residual: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """residual + x (rounded once to the activation dtype) and its norm; ``residual`` may be updated in place."""
        raise NotImplementedError


class Mixer(Part):
    # True for a mixer with state of its own whose call reads the step's device tables only (``state_slots``, ``token_row``,
    # ``positions``, ``q_indptr`` ...), never host values: a step is the same sequence of launches whatever its rows are,
    # so the executor may capture it. The default keeps such a model's steps eager (a mixer written as a Python loop over
    # the rows is then right as it is).
    state_capturable = False

    def cache_need(self) -> CacheNeed | None:
        return None

    # ---- per-step work lists (optional). A mixer whose kernels want lists derived on the host from the step's rows
    # (how the rows are divided among kernels and CTAs) asks the batch for them in its call: ``batch.step_work(self,
    # key)``. The batch calls back here. Neither the batch nor the executor knows what the lists hold: a captured step
    # sizes its fixed tables with ``step_work_caps``, refills them with ``step_work_arrays`` before every replay and lets
    # the mixer bind them once, at capture, with ``step_work_bind``. ``key`` is any hashable that starts with the mixer's
    # kind; runs that ask under the same key share one set of lists.
    def step_class(self, row_counts: list) -> tuple:
        """What about a step's rows decides which lists the step needs at all (part of a captured step's identity)."""
        return ()

    def step_work_arrays(self, key, row_starts: list, row_counts: list) -> list:
        """The step's lists as int32 numpy arrays. A padding row has start -1."""
        raise NotImplementedError

    def step_work_caps(self, key, num_tokens: int, num_rows: int, kv_cap: int, step_class: tuple) -> list:
        """(capacity, fill value) of each list for a captured step of these sizes; entries beyond a step's own are set to
        the fill value, which the kernels must skip."""
        raise NotImplementedError

    def step_work_bind(self, key, tensors: list, host_arrays: list | None = None, captured: tuple | None = None):
        """What the mixer's call gets back from ``batch.step_work``: built from the lists on the device and either the
        host arrays they were copied from (an eager step) or, in a captured step whose tables have their full capacity,
        ``captured`` = (num_tokens, num_rows, kv_cap, step_class)."""
        raise NotImplementedError

    def __call__(self, x: torch.Tensor, batch, cache, write_cache: bool = True) -> torch.Tensor:
        """x: [T, hidden] normed input of this step's tokens. ``batch`` is the step's ``StepBatch``; ``cache``
        is this run's view of its cache group (None when ``cache_need`` is None). With ``write_cache`` False
        the run reads another run's cache and must not write it. In a captured step the batch may end in padding
        rows: tokens at position -1 of a row that holds no keys (``kv_lens`` 0, an empty page range, slot -1); nothing is
        written to the cache for them and nobody reads their output."""
        raise NotImplementedError


class FeedForward(Part):
    def __call__(self, x: torch.Tensor, batch) -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    """Token ids to the first hidden states. Declares its parameters under the scope "embed"; ``tied_weight`` is what a
    head that shares the embedding's matrix is loaded with (None when the part has nothing to share)."""

    def __call__(self, ids: torch.Tensor, batch) -> torch.Tensor:
        """ids: int32 [T]; returns [T, hidden] in the activation dtype."""
        raise NotImplementedError

    def tied_weight(self) -> torch.Tensor | None:
        return None


class Head(Part):
    """The final hidden states of the wanted rows to float32 logits [rows, vocab]. Declares its parameters under the scope
    "lm_head"; with tied embeddings it declares none and is loaded with {"weight": the embedding's ``tied_weight``}."""

    def __call__(self, final: torch.Tensor, batch) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer

    def __call__(self, h, residual, batch, cache, write_cache: bool = True):
        """(h, residual) in, (h, residual) out; ``residual`` is None before the first block."""
        raise NotImplementedError

    def sub_parts(self) -> dict[str, Part]:
        raise NotImplementedError


class _Registry:
    def __init__(self, what: str):
        self.what = what
        self._kinds: dict[str, Callable] = {}

    def register(self, kind: str, cls) -> None:
        self._kinds[kind] = cls

    def get(self, kind: str):
        try:
            return self._kinds[kind]
        except KeyError:
            raise KeyError(f"no {self.what} of kind '{kind}' is registered (registered: {', '.join(sorted(self._kinds)) or 'none'})") from None

    def build(self, spec, runtime: Runtime):
        return self.get(spec.kind)(spec, runtime)


NORMS = _Registry("norm")
POSITIONS = _Registry("position encoding")
MIXERS = _Registry("mixer")
FEED_FORWARDS = _Registry("feed-forward")
BLOCKS = _Registry("block arrangement")
EMBEDDINGS = _Registry("embedding")
HEADS = _Registry("head")


def register_norm(kind, cls):
    NORMS.register(kind, cls)


def register_position(kind, cls):
    POSITIONS.register(kind, cls)


def register_mixer(kind, cls):
    MIXERS.register(kind, cls)


def register_feed_forward(kind, cls):
    FEED_FORWARDS.register(kind, cls)


def register_block(kind, cls):
    BLOCKS.register(kind, cls)


def register_embedding(kind, cls):
    EMBEDDINGS.register(kind, cls)


def register_head(kind, cls):
    HEADS.register(kind, cls)
