"""Device memory of the cache groups.

A paged group is one tensor [runs, planes, pages, kv_heads, page_size, head_dim] in the compute dtype (planes: keys and
values, or the one tensor of a group whose mixers keep a single vector a token): a page id
addresses the page of every run in the group, as the reference's "bytes per block across all layers" does
(src/Starlings.Roost.Abstractions/State/StateGroups.cs:83-84); within a page the layout is head-major so that
one head's keys of a page are contiguous. A state group is one tensor [runs, slots + 1, *state_shape]: the last slot
belongs to no request and takes what the padding rows of a captured step write.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .manager import CacheGroup


@dataclass
class CacheView:
    """What one run of a mixer sees of its cache."""
    group: int                        # index of the group: selects the batch's tables
    kind: str
    page_size: int = 0
    k_pool: torch.Tensor | None = None   # [pages, kv_heads, page_size, head_dim]; the only pool of a group with one plane
    v_pool: torch.Tensor | None = None
    state: torch.Tensor | None = None    # [slots, *state_shape]


class CacheStorage:
    def __init__(self, groups: list[CacheGroup], capacities: list[int], dtype: torch.dtype, device):
        self.groups = groups
        self.tensors = []
        self._view_of_run: dict[int, CacheView] = {}
        for gi, (g, cap) in enumerate(zip(groups, capacities)):
            if g.kind == "paged":
                t = torch.zeros((max(len(g.runs), 1), g.planes, cap, g.kv_heads, g.page_size, g.head_dim), dtype=dtype, device=device)
                for li, run in enumerate(g.runs):
                    self._view_of_run[run] = CacheView(group=gi, kind="paged", page_size=g.page_size, k_pool=t[li, 0],
                                                       v_pool=t[li, 1] if g.planes == 2 else None)
            else:
                # one slot more than the pool hands out: the scratch slot that the padding rows of a captured step name
                t = torch.zeros((max(len(g.runs), 1), cap + 1, *g.state_shape), dtype=g.state_dtype, device=device)
                for li, run in enumerate(g.runs):
                    self._view_of_run[run] = CacheView(group=gi, kind="state", state=t[li])
            self.tensors.append(t)

    def view(self, run: int) -> CacheView | None:
        return self._view_of_run.get(run)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors)

    def poison(self, value: float = float("nan")) -> None:
        """Fills every page with a value that shows if a kernel reads a slot nobody wrote (tests)."""
        for g, t in zip(self.groups, self.tensors):
            if g.kind == "paged":
                t.fill_(value)
