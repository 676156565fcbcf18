"""Sampling above the step function: greedy, or temperature with top-k, top-p and min-p, on the device.

One call samples every row of a step that wants a token. A batch of greedy rows goes to the argmax kernel;
otherwise the per-row parameter tables are uploaded in one copy and the sampling kernel runs (greedy rows in
such a batch are rows with temperature 0). The draw of a row depends on its own seed and on how many tokens
its request has generated (the Philox offset), not on the batch or the row index, so a request that is
preempted and recomputed draws the same tokens again
(src/Starlings.Roost.Engine/Scheduling/StepPlanner.cs:955-968, src/Starlings.Roost.Ops/CpuOps.Sampling.cs:39-41).
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


class Sampler:
    def __init__(self, kernels, device):
        self.kernels = kernels
        self.device = torch.device(device)
        self._workspace: torch.Tensor | None = None

    def __call__(self, logits: torch.Tensor, rows: list[SamplingRow]) -> torch.Tensor:
        """logits [S, vocab] float32 on the device; returns int32 token ids [S] on the device."""
        if logits.shape[0] != len(rows):
            raise ValueError(f"{logits.shape[0]} rows of logits for {len(rows)} sampling rows")
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
