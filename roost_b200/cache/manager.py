"""The cache manager: which pages and state slots every live request holds.

Runs of mixers are sorted into groups by what they keep between steps (``CacheNeed``): paged keys and values
of one geometry with every earlier token, paged with a window, or a fixed-size state per request. Each paged
group has a pool of page ids of its own and a block table per request (index = position // page size; a page
that a window has passed is given back and its entry becomes ``NULL_PAGE``); one page id addresses the page of
every run in the group. Each state group has a pool of slots, one per live request. The reference's state
groups are the model for this (src/Starlings.Roost.Abstractions/State/StateGroups.cs:9-37,63-100), its planner
takes pages for the rows it is about to run and never ahead (src/Starlings.Roost.Engine/Scheduling/
StepPlanner.cs:741-751,772-788), and gives them back when a request finishes or is preempted (:978-1023).

This module is host-side bookkeeping only; ``storage.py`` owns the device tensors.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .block_pool import NULL_PAGE, BlockPool, PoolError


class OutOfPages(RuntimeError):
    """A request needs more pages or slots than its pools have free."""


@dataclass(frozen=True)
class CacheGroup:
    name: str
    kind: str                      # "paged" | "state"
    runs: tuple                    # indices of the schedule entries whose cache lives in this group
    page_size: int = 0
    window: int | None = None      # keys a query sees, its own included; None = all
    kv_heads: int = 0
    head_dim: int = 0
    planes: int = 2                # tensors kept per token: keys and values, or one
    state_shape: tuple = ()
    state_dtype: torch.dtype = torch.float32

    def bytes_per_page(self, element_size: int) -> int:
        return self.planes * len(self.runs) * self.page_size * self.kv_heads * self.head_dim * element_size


def leading_releasable_pages(tokens: int, window: int, page_size: int) -> int:
    """Pages whose every position lies below ``tokens - window``: one position more is kept than a window
    of ``window`` keys that includes the query needs, so no page a later query can read is released
    (src/Starlings.Roost.Engine/Blocks/BlockPool.cs:255-270)."""
    return (tokens - window) // page_size if tokens > window else 0


@dataclass
class RequestCache:
    request_id: object
    tokens: int = 0                                   # tokens whose keys/values (or state) are in the cache
    tables: list = field(default_factory=list)        # per group: list of page ids (paged) or None
    slots: list = field(default_factory=list)         # per group: slot id (state) or None


class CacheManager:
    def __init__(self, groups: list[CacheGroup], capacities: list[int]):
        """``capacities``: pages per paged group, slots per state group, in the order of ``groups``."""
        if len(groups) != len(capacities):
            raise ValueError("one capacity per cache group is needed")
        self.groups = list(groups)
        self.pools = [BlockPool(c, name=g.name) for g, c in zip(groups, capacities)]
        self._requests: dict[object, RequestCache] = {}

    # ------------------------------------------------------------------ queries
    def __contains__(self, request_id) -> bool:
        return request_id in self._requests

    def get(self, request_id) -> RequestCache:
        try:
            return self._requests[request_id]
        except KeyError:
            raise KeyError(f"request {request_id!r} holds no cache") from None

    @property
    def live_requests(self):
        return self._requests.keys()

    def pages_needed(self, request_id, new_total: int) -> list[int]:
        """Per group, how many more pages (or slots) the request needs to hold ``new_total`` tokens."""
        rc = self._requests.get(request_id)
        need = []
        for gi, g in enumerate(self.groups):
            if g.kind == "state":
                need.append(0 if rc is not None else 1)
            else:
                have = len(rc.tables[gi]) if rc is not None else 0
                need.append(max(0, -(-new_total // g.page_size) - have))
        return need

    def can_hold(self, request_id, new_total: int, extra_free: list[int] | None = None) -> bool:
        need = self.pages_needed(request_id, new_total)
        return all(n <= self.pools[gi].free_count + (extra_free[gi] if extra_free else 0) for gi, n in enumerate(need))

    def held(self, request_id) -> list[int]:
        """Per group, pages (or slots) the request holds now."""
        rc = self._requests.get(request_id)
        if rc is None:
            return [0] * len(self.groups)
        return [1 if g.kind == "state" else sum(1 for p in rc.tables[gi] if p != NULL_PAGE) for gi, g in enumerate(self.groups)]

    def max_tokens_per_request(self) -> int:
        """The longest request the paged pools could ever hold alone (window groups bound nothing)."""
        caps = [self.pools[gi].capacity * g.page_size for gi, g in enumerate(self.groups) if g.kind == "paged" and g.window is None]
        return min(caps) if caps else 1 << 60

    def usage(self) -> float:
        tot = sum(p.capacity for g, p in zip(self.groups, self.pools) if g.kind == "paged")
        used = sum(p.used_count for g, p in zip(self.groups, self.pools) if g.kind == "paged")
        return used / tot if tot else 0.0

    # ------------------------------------------------------------------ changes
    def extend(self, request_id, new_total: int) -> RequestCache:
        """Takes the pages the request needs to hold ``new_total`` tokens (and, for a request seen for the
        first time, its state slots). All or none: on ``OutOfPages`` nothing has changed."""
        rc = self._requests.get(request_id)
        if rc is not None and new_total < rc.tokens:
            raise ValueError(f"request {request_id!r} already holds {rc.tokens} tokens; cannot shrink to {new_total}")
        need = self.pages_needed(request_id, new_total)
        for gi, n in enumerate(need):
            if n > self.pools[gi].free_count:
                g = self.groups[gi]
                raise OutOfPages(f"group '{g.name}' has {self.pools[gi].free_count} free of {self.pools[gi].capacity}; "
                                 f"request {request_id!r} needs {n} more to hold {new_total} tokens")
        if rc is None:
            rc = RequestCache(request_id, 0, [[] if g.kind == "paged" else None for g in self.groups],
                              [None] * len(self.groups))
            self._requests[request_id] = rc
        for gi, (g, n) in enumerate(zip(self.groups, need)):
            if n == 0:
                continue
            got = self.pools[gi].try_allocate(n)
            assert got is not None
            if g.kind == "state":
                rc.slots[gi] = got[0]
            else:
                rc.tables[gi].extend(got)
        return rc

    def commit(self, request_id, new_total: int) -> int:
        """Records that the cache now holds ``new_total`` tokens of the request and gives back the pages a
        window has passed. Returns how many pages were released."""
        rc = self.get(request_id)
        rc.tokens = new_total
        released = 0
        for gi, g in enumerate(self.groups):
            if g.kind != "paged" or g.window is None:
                continue
            table = rc.tables[gi]
            n = min(leading_releasable_pages(new_total, g.window, g.page_size), len(table))
            for i in range(n):
                if table[i] != NULL_PAGE:
                    self.pools[gi].release(table[i])
                    table[i] = NULL_PAGE
                    released += 1
        return released

    def free(self, request_id) -> None:
        """Gives back everything the request holds. Freed pages go to the top of their pool's stack in
        reverse table order, so the next request takes them first."""
        rc = self._requests.pop(request_id, None)
        if rc is None:
            return
        for gi, g in enumerate(self.groups):
            if g.kind == "state":
                if rc.slots[gi] is not None:
                    self.pools[gi].release(rc.slots[gi])
            else:
                for p in reversed(rc.tables[gi]):
                    if p != NULL_PAGE:
                        self.pools[gi].release(p)

    def free_all(self) -> None:
        for rid in list(self._requests):
            self.free(rid)

    # ------------------------------------------------------------------ checks
    def check_invariants(self) -> None:
        """No page lost, held twice or free while held; pool counts agree with the tables."""
        for gi, (g, pool) in enumerate(zip(self.groups, self.pools)):
            pool.check_invariants()
            held = {}
            for rc in self._requests.values():
                ids = [rc.slots[gi]] if g.kind == "state" else [p for p in rc.tables[gi] if p != NULL_PAGE]
                for p in ids:
                    if p is None:
                        raise PoolError(f"group '{g.name}': request {rc.request_id!r} has no slot")
                    if p in held:
                        raise PoolError(f"group '{g.name}': page {p} is held by {held[p]!r} and {rc.request_id!r}")
                    if pool.refs(p) != 1:
                        raise PoolError(f"group '{g.name}': page {p} of {rc.request_id!r} has count {pool.refs(p)}")
                    held[p] = rc.request_id
            if len(held) != pool.used_count:
                raise PoolError(f"group '{g.name}': {pool.used_count} pages are taken but requests hold {len(held)} (a page is lost)")


def build_groups(needs: list, page_size: int) -> list[CacheGroup]:
    """Sorts the schedule's runs into groups. ``needs[i]`` is the ``CacheNeed`` of run i, or None when the run
    keeps nothing or reads another run's cache. Paged runs with the same (window, kv_heads, head_dim, planes) share a
    group; every state run with the same shape and dtype shares one. A group of fixed-size state always exists,
    with no runs and a zero-sized state when the model has none, so that slots are handed out and returned on
    every path."""
    paged: dict[tuple, list[int]] = {}
    state: dict[tuple, list[int]] = {}
    for i, need in enumerate(needs):
        if need is None:
            continue
        if need.kind == "paged":
            if need.planes not in (1, 2):
                raise ValueError(f"run {i} asks for {need.planes} tensors a token; a paged cache keeps 1 or 2")
            paged.setdefault((need.window, need.kv_heads, need.head_dim, need.planes), []).append(i)
        elif need.kind == "state":
            state.setdefault((tuple(need.state_shape), need.state_dtype), []).append(i)
        else:
            raise ValueError(f"run {i} asks for a cache of kind '{need.kind}'")
    groups = []
    for (window, kvh, d, planes), runs in paged.items():
        name = ("full" if window is None else f"window{window}") + f"_h{kvh}d{d}" + ("" if planes == 2 else f"x{planes}")
        groups.append(CacheGroup(name=name, kind="paged", runs=tuple(runs), page_size=page_size, window=window,
                                 kv_heads=kvh, head_dim=d, planes=planes))
    for (shape, dt), runs in state.items():
        groups.append(CacheGroup(name="state" + "x".join(map(str, shape)), kind="state", runs=tuple(runs),
                                 state_shape=shape, state_dtype=dt))
    if not state:
        groups.append(CacheGroup(name="state_none", kind="state", runs=(), state_shape=(0,)))
    return groups
