"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

``StepExecutor.step`` runs only the tokens it is given, as one batch, against the cache that earlier steps
left: it takes the pages the rows need, builds the step's tables, runs the model's forward pass once and
records the new lengths (which also gives back pages that a window has passed). It samples nothing and keeps
no request state beyond what the cache manager holds. Generation, the replay tool and the tests all drive
this one function. The reference's worker has the same shape: plan in, one forward pass over mixed rows,
logits of the selected rows out (src/Starlings.Roost.Worker/Eager/EagerWorker.cs:193-283), with every index
checked on the host before anything is launched (src/Starlings.Roost.Worker/Eager/StepPlanReader.cs:168-356).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..cache.manager import CacheManager, OutOfPages, build_groups
from ..cache.storage import CacheStorage
from .batch import BatchBuilder
from .model import Model


@dataclass
class StepEntry:
    """One row of a step: the request's next tokens and the offsets among them whose logits are wanted."""
    request_id: object
    tokens: list
    want: list = field(default_factory=list)
    start: int | None = None     # the position the caller believes the first token has; checked when given


class StepError(ValueError):
    """A step that was refused before anything was launched."""


class StepExecutor:
    def __init__(self, model: Model, *, page_size: int = 16, num_pages: int | None = None, max_tokens: int | None = None,
                 max_requests: int = 64, kv_fraction: float = 0.9):
        """``num_pages`` per paged group, or ``max_tokens`` (the most tokens live requests hold at any time,
        rounded up to whole pages), or else ``kv_fraction`` of the device memory that is free now."""
        if page_size <= 0:
            raise ValueError(f"page size {page_size} must be positive")
        self.model = model
        self.rt = model.rt
        self.page_size = page_size
        self.groups = build_groups(model.cache_needs, page_size)
        elem = torch.empty((), dtype=self.rt.dtype).element_size()
        if num_pages is None and max_tokens is not None:
            num_pages = -(-max_tokens // page_size)
        if num_pages is None:
            per_page = sum(g.bytes_per_page(elem) for g in self.groups if g.kind == "paged")
            free, _ = torch.cuda.mem_get_info(self.rt.device)
            num_pages = max(1, int(free * kv_fraction) // max(per_page, 1))
        self.num_pages = num_pages
        capacities = [num_pages if g.kind == "paged" else max_requests for g in self.groups]
        self.cache = CacheManager(self.groups, capacities)
        self.storage = CacheStorage(self.groups, capacities, self.rt.dtype, self.rt.device)
        self.builder = BatchBuilder(self.rt.device, self.cache)
        self.steps_run = 0
        self.last_upload_bytes = 0

    # ------------------------------------------------------------------ one step
    def step(self, entries: list[StepEntry]) -> torch.Tensor:
        """Logits [wanted, vocab] float32 on the device, in the order of the entries and of their ``want``."""
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        plan = []
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request_id!r} brings no tokens")
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"request {e.request_id!r} wants offset {w} among {n} tokens")
            start = self.cache.get(e.request_id).tokens if e.request_id in self.cache else 0
            if e.start is not None and e.start != start:
                raise StepError(f"request {e.request_id!r}: the row starts at position {e.start} but the cache holds {start} tokens")
            plan.append((e, start, start + n))
        max_pos = self.model.spec.max_positions
        if max_pos:
            for e, _, end in plan:
                if end > max_pos:
                    raise StepError(f"request {e.request_id!r} would reach {end} tokens; the model has {max_pos} positions")
        # all-or-none over the step: check the total need first
        need = [0] * len(self.groups)
        for e, _, end in plan:
            for gi, n in enumerate(self.cache.pages_needed(e.request_id, end)):
                need[gi] += n
        for gi, n in enumerate(need):
            if n > self.cache.pools[gi].free_count:
                raise OutOfPages(f"group '{self.groups[gi].name}': the step needs {n} more pages or slots, {self.cache.pools[gi].free_count} are free")
        rows = []
        new_requests = []
        for e, start, end in plan:
            if e.request_id not in self.cache:
                new_requests.append(e.request_id)
            rc = self.cache.extend(e.request_id, end)
            rows.append((rc, start, e.tokens, e.want))
        try:
            batch = self.builder.build(rows, self.model.spec.vocab)
        except Exception:
            for rid in new_requests:
                self.cache.free(rid)
            raise
        self.last_upload_bytes = batch.host_buffer.numel() * batch.host_buffer.element_size()
        self._zero_new_state(rows)
        logits = self.model.forward(batch, self.storage)
        for (e, _, end) in plan:
            self.cache.commit(e.request_id, end)
        self.steps_run += 1
        return logits

    def _zero_new_state(self, rows) -> None:
        """A request's fixed-size state starts at zero when its first token arrives, as the reference's worker
        zeroes a recurrent slot at position 0 (src/Starlings.Roost.Worker/Eager/EagerWorker.cs:214-230)."""
        for gi, g in enumerate(self.groups):
            if g.kind != "state" or not g.runs:
                continue
            fresh = [rc.slots[gi] for rc, start, _, _ in rows if start == 0]
            if fresh:
                idx = torch.tensor(fresh, dtype=torch.long, device=self.rt.device)
                self.storage.tensors[gi].index_fill_(1, idx, 0)

    def finish(self, request_id) -> None:
        """The request is done: everything it holds goes back to the pools."""
        self.cache.free(request_id)

    def tokens_cached(self, request_id) -> int:
        return self.cache.get(request_id).tokens if request_id in self.cache else 0
