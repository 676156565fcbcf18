"""The arrangement of a layer's parts. ``pre_norm``: h += mixer(norm1(h)); h += feed_forward(norm2(h))
(src/Starlings.Roost.Models.Tiny/RoostTiny.cs:40,49-50,54). The residual stream is carried beside the branch
output so that each residual sum is fused into the norm that follows it; the stream is stored in the
activation dtype and every sum is formed in 32-bit and rounded once."""
from __future__ import annotations

from ..config.spec import BlockSpec
from .base import FEED_FORWARDS, MIXERS, NORMS, Block, Runtime, register_block


class PreNormBlock(Block):
    def __init__(self, spec: BlockSpec, runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        self.input_norm = NORMS.build(spec.input_norm, runtime)
        self.mixer = MIXERS.build(spec.mixer, runtime)
        self.post_mixer_norm = NORMS.build(spec.post_mixer_norm, runtime)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, runtime)

    def sub_parts(self):
        return {"input_norm": self.input_norm, "mixer": self.mixer, "post_mixer_norm": self.post_mixer_norm,
                "feed_forward": self.feed_forward}

    @classmethod
    def sub_specs(cls, spec: BlockSpec):
        return {"input_norm": (NORMS, spec.input_norm), "mixer": (MIXERS, spec.mixer),
                "post_mixer_norm": (NORMS, spec.post_mixer_norm), "feed_forward": (FEED_FORWARDS, spec.feed_forward)}

    def __call__(self, h, residual, batch, cache, write_cache: bool = True):
        """``h`` is the previous branch output (or the embedding), ``residual`` the stream before it was added
        (None at the first block). Returns the feed-forward's output and the stream it is still to be added to."""
        if residual is None:
            residual = h
            x = self.input_norm(h)
        else:
            x, residual = self.input_norm.add_norm(h, residual)
        a = self.mixer(x, batch, cache, write_cache)
        y, residual = self.post_mixer_norm.add_norm(a, residual)
        return self.feed_forward(y, batch), residual


register_block("pre_norm", PreNormBlock)
