"""The two ends of a model: the token embedding and the head that turns final hidden states into logits.

``table``: h0[t, :] = table[ids[t], :], a bit-exact row copy with no scaling (src/Starlings.Roost.Ops/CpuOps.cs:441-458).
``linear``: logits[s, v] = sum_d final[s, d] W[v, d] in 32-bit whatever the activation dtype is, no soft cap
(src/Starlings.Roost.Ops/CpuOps.cs:465-495); with tied embeddings W is the embedding's table. An architecture that scales
its embeddings or caps its logits registers other kinds; the model only knows the two interfaces.
"""
from __future__ import annotations

import torch

from ..config.spec import EmbeddingSpec, HeadSpec
from .base import Embedding, Head, ParamDecl, Runtime, register_embedding, register_head
from .linear import Linear


class TableEmbedding(Embedding):
    def __init__(self, spec: EmbeddingSpec, runtime: Runtime):
        if spec.vocab <= 0 or spec.hidden <= 0:
            raise ValueError("table embedding: vocab and hidden must be positive")
        self.spec, self.rt = spec, runtime
        self.table: torch.Tensor | None = None

    @classmethod
    def parameters(cls, spec: EmbeddingSpec):
        return {"table": ParamDecl(shape=(spec.vocab, spec.hidden))}

    def load(self, params):
        self.table = params["table"].to(self.rt.dtype).contiguous()

    def tied_weight(self):
        return self.table

    def __call__(self, ids, batch=None):
        return self.rt.kernels.embedding(self.table, ids)


class LinearHead(Head):
    def __init__(self, spec: HeadSpec, runtime: Runtime):
        self.spec, self.rt = spec, runtime
        self.linear = Linear(runtime, spec.vocab, spec.hidden)

    @classmethod
    def parameters(cls, spec: HeadSpec):
        return {"weight": ParamDecl(shape=(spec.vocab, spec.hidden))}

    def load(self, params):
        w = params["weight"]
        if w.dtype == self.rt.dtype and w.is_contiguous() and tuple(w.shape) == (self.spec.vocab, self.spec.hidden):
            self.linear.weight = w          # as it is: a tied head shares the embedding's memory
        else:
            self.linear.load(w)

    @property
    def weight(self):
        return self.linear.weight

    def __call__(self, final, batch=None):
        return self.linear(final, out_dtype=torch.float32)


register_embedding("table", TableEmbedding)
register_head("linear", LinearHead)
