"""Position encodings a mixer can be given.

The attention mixer's fused kernel rotates the first ``rotary_dim`` elements of every query and key head by
the angle position * inv_freq[i], pairing element i with i + rotary_dim/2 (NeoX form,
src/Starlings.Roost.Ops/CpuOps.cs:111-177). A position encoding therefore hands the mixer a table of
frequencies in double precision and a rotary width; ``rotary_dim`` 0 means no rotation. Frequency-scaled
variants are other tables behind the same interface. An encoding whose angles are not position x frequency (several
position axes, angles looked up in a table) gives the step's cosines and sines itself (``step_table``); the pairing of
elements stays the kernel's.
"""
from __future__ import annotations

import torch

from ..config.spec import PositionSpec
from .base import Part, Runtime, register_position


class PositionEncoding(Part):
    def rotation(self) -> tuple[torch.Tensor | None, int]:
        """(inv_freq: float64 [rotary_dim / 2] on the device, rotary_dim)."""
        raise NotImplementedError

    def step_table(self, batch) -> torch.Tensor | None:
        """Optional: the cosines and sines of this step's tokens, float32 [T, rotary_dim / 2, 2] on the device, made from
        the step's device tables (``batch.positions``: -1 for the padding tokens of a captured step). None (the default):
        the kernels form position * inv_freq themselves."""
        return None

    max_positions: int = 0  # 0: unbounded


_FREQUENCIES: dict = {}   # (theta, rotary_dim, device) -> the frequency table that equal encodings share


class RopeNeox(PositionEncoding):
    """f_i = theta^(-2i / rotary_dim), computed in double once at build. Encodings of equal theta and width on one device
    hand out the same tensor: a step keeps its table of cosines and sines by that tensor, so that the layers of a model,
    each with an encoding of its own, share one table a step."""

    def __init__(self, spec: PositionSpec, runtime: Runtime):
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError(f"rope_neox: rotary_dim {spec.rotary_dim} must be positive and even")
        if spec.theta <= 0:
            raise ValueError(f"rope_neox: theta {spec.theta} must be positive")
        self.spec = spec
        self.max_positions = spec.max_positions
        key = (float(spec.theta), spec.rotary_dim, str(torch.device(runtime.device)))
        if key not in _FREQUENCIES:
            i = torch.arange(spec.rotary_dim // 2, dtype=torch.float64)
            _FREQUENCIES[key] = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * i / spec.rotary_dim).to(runtime.device)
        self.inv_freq = _FREQUENCIES[key]

    def rotation(self):
        return self.inv_freq, self.spec.rotary_dim


class NoPosition(PositionEncoding):
    def __init__(self, spec: PositionSpec, runtime: Runtime):
        self.spec = spec

    def rotation(self):
        return None, 0


register_position("rope_neox", RopeNeox)
register_position("none", NoPosition)
