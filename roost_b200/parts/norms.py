"""RMS norm: y = x / sqrt(mean(x^2) + eps) * w with the weight as stored
(src/Starlings.Roost.Ops/CpuOps.cs:87-101), alone or fused with the residual sum that precedes it
(src/Starlings.Roost.Ops/CpuOps.Fused.cs:26-34)."""
from __future__ import annotations

import torch

from ..config.spec import NormSpec
from .base import Norm, ParamDecl, Runtime, register_norm


class RmsNorm(Norm):
    def __init__(self, spec: NormSpec, runtime: Runtime):
        if spec.size <= 0 or spec.eps <= 0:
            raise ValueError(f"rms_norm: size {spec.size} and eps {spec.eps} must be positive")
        self.spec = spec
        self.rt = runtime
        self.weight: torch.Tensor | None = None

    @classmethod
    def parameters(cls, spec: NormSpec):
        return {"weight": ParamDecl(shape=(spec.size,), role="vector")}

    def load(self, params):
        self.weight = params["weight"].contiguous()

    def __call__(self, x: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        return self.rt.kernels.rms_norm(x, self.weight, self.spec.eps, rows)

    def add_norm(self, x: torch.Tensor, residual: torch.Tensor, rows: torch.Tensor | None = None):
        """Returns (norm(residual + x), residual + x); without ``rows`` the sum replaces ``residual`` in place."""
        out = self.rt.kernels.add_rms_norm(x, residual, self.weight, self.spec.eps, rows)
        return out, residual


register_norm("rms_norm", RmsNorm)
