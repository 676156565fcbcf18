"""The gated feed-forward: down(act(x Wg^T) * (x Wu^T)), gate and up as one product over the row-wise
concatenation [gate; up] made at load (src/Starlings.Roost.Models.Tiny/RoostTiny.cs:35-36,51-53;
silu(g) = g / (1 + exp(-g)), src/Starlings.Roost.Ops/CpuOps.cs:355-368)."""
from __future__ import annotations

from ..config.spec import GatedMlpSpec
from .base import FeedForward, ParamDecl, Runtime, register_feed_forward
from .linear import Linear


class GatedMlp(FeedForward):
    def __init__(self, spec: GatedMlpSpec, runtime: Runtime):
        if spec.hidden <= 0 or spec.intermediate <= 0:
            raise ValueError("gated_mlp: hidden and intermediate must be positive")
        if spec.activation != "silu":
            raise ValueError(f"gated_mlp: activation '{spec.activation}' has no kernel (built: silu)")
        self.spec = spec
        self.rt = runtime
        self.gate_up = Linear(runtime, 2 * spec.intermediate, spec.hidden)
        self.down = Linear(runtime, spec.hidden, spec.intermediate)

    @classmethod
    def parameters(cls, spec: GatedMlpSpec):
        I, H = spec.intermediate, spec.hidden
        return {"gate_up": ParamDecl(shape=(2 * I, H), row_splits=(I, I)), "down": ParamDecl(shape=(H, I))}

    def load(self, params):
        self.gate_up.load(params["gate_up"])
        self.down.load(params["down"])

    def __call__(self, x, batch=None):
        return self.down(self.rt.kernels.silu_mul(self.gate_up(x)))


register_feed_forward("gated_mlp", GatedMlp)
