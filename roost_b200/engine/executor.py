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

import weakref
from dataclasses import dataclass, field

import torch

import numpy as np

from ..cache.manager import CacheManager, OutOfPages, build_groups
from ..cache.storage import CacheStorage
from .batch import AttentionPlan, BatchBuilder, HostTables, StaticTables, attention_caps, attention_work
from .model import Model

GRAPH_KV_GRANULE = 1024   # a captured decode step serves requests of up to a multiple of this many tokens
MAX_GRAPHS = 24


@dataclass
class StepEntry:
    """One row of a step: the request's next tokens and the offsets among them whose logits are wanted."""
    request_id: object
    tokens: list
    want: list = field(default_factory=list)
    start: int | None = None     # the position the caller believes the first token has; checked when given


class StepError(ValueError):
    """A step that was refused before anything was launched."""


@dataclass
class PreparedDecode:
    """The tables of a decode step made before its token ids are known (see ``StepExecutor.prepare_decode``)."""
    request_ids: list
    starts: list
    graph: object
    staged: int       # the pinned buffer of the graph's tables that holds this step's tables; section 0 is the token ids


class DecodeGraph:
    """A captured CUDA graph of one decode step (every row brings one token and wants its logits) for a fixed number
    of rows and a bound on the requests' lengths. The step's tables live at fixed device addresses; a replay uploads
    the new tables and launches the whole forward pass with one call, so the host's per-kernel launch cost (hundreds
    of launches a step) no longer bounds small batches. The reference's one graph experiment did not replay
    bit-identically and is unclaimed (kernels/README.md:240-250); here a replay runs the very kernels of the eager
    path with the same arguments, and the tests compare both with the plain implementation."""

    def __init__(self, executor: "StepExecutor", num_rows: int, kv_cap: int, plan_keys: list):
        self.ex = weakref.proxy(executor)   # the executor owns its graphs; no reference cycle keeps its cache alive
        self.num_rows, self.kv_cap = num_rows, kv_cap
        self.plan_keys = list(plan_keys)
        builder = executor.builder
        table_caps = builder.table_caps(num_rows, kv_cap)
        self.n_table = len(table_caps)
        self.plan_caps = [attention_caps(num_rows, kv_cap, g, chunk, rows) for (g, _w, chunk, rows) in self.plan_keys]
        caps, fills = list(table_caps), [0] * len(table_caps)
        for pc, dc, mc in self.plan_caps:
            caps += [pc * 2, dc * 4, mc * 4]
            fills += [-1, -1, -1]    # padding items name batch row -1, which the kernels skip
        self.fills = fills
        self.static = StaticTables(executor.rt.device, caps)
        self.graph = None
        self.out = None

    def _arrays(self, ht: HostTables) -> list:
        arrays = list(ht.arrays)
        for (g, w, chunk, rows) in self.plan_keys:
            prefill, decode, merge, _ = attention_work(ht.row_starts, ht.row_counts, g, w, chunk, rows)
            arrays += [np.asarray(prefill, np.int32), np.asarray(decode, np.int32), np.asarray(merge, np.int32)]
        return arrays

    def fits(self, ht: HostTables) -> bool:
        self._pending = self._arrays(ht)
        return self.static.fits(self._pending)

    def run(self, ht: HostTables) -> torch.Tensor:
        """Call after ``fits(ht)`` returned True."""
        self.static.upload(self._pending, self.fills)
        if self.graph is None:
            return self._capture(ht)
        self.graph.replay()
        self.ex.rt.kernels.launches += self.launches
        return self.out.clone()

    def run_staged(self, staged: int) -> torch.Tensor:
        """A replay with tables staged earlier (the graph is captured already)."""
        self.static.send(staged)
        self.graph.replay()
        self.ex.rt.kernels.launches += self.launches
        return self.out.clone()

    def _capture(self, ht: HostTables) -> torch.Tensor:
        ex = self.ex
        batch = ex.builder.static_batch(ht, self.static, self.n_table)
        views = self.static.views[self.n_table:]
        for i, (key, (pc, dc, mc)) in enumerate(zip(self.plan_keys, self.plan_caps)):
            batch.attention_plans[key] = AttentionPlan(prefill_items=pc, prefill_tile_rows=key[3], decode_items=dc, merge_items=mc, slots=dc,
                                                       merge_rows=min(16, key[0]),   # one token a row: its query heads per key/value head
                                                       prefill_work=views[3 * i], decode_work=views[3 * i + 1],
                                                       merge_work=views[3 * i + 2])
        # this step's result comes from an eager run on a side stream (which also warms every kernel and library up);
        # the capture that follows records the same launches without running them
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            result = ex.model.forward(batch, ex.storage).clone()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        before = ex.rt.kernels.launches
        with torch.cuda.graph(graph):
            out = ex.model.forward(batch, ex.storage)
        self.launches = ex.rt.kernels.launches - before   # kernels one replay launches
        ex.rt.kernels.launches = before
        self.graph, self.out, self.batch = graph, out, batch
        return result


class StepExecutor:
    def __init__(self, model: Model, *, page_size: int = 16, num_pages: int | None = None, max_tokens: int | None = None,
                 max_requests: int = 64, kv_fraction: float = 0.9, use_graphs: bool = True):
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
        # decode steps are replayed from captured graphs when every run keeps paged keys and values only (a mixer with
        # state of its own may be written in Python and may not be idempotent, so such models run eagerly) and every
        # part says that its call can be captured
        self.use_graphs = (use_graphs and self.rt.device.type == "cuda"
                           and all(g.kind == "paged" or not g.runs for g in self.groups)
                           and all(getattr(p, "capturable", True) for p in model.parts()))
        self._graphs: dict = {}
        self._plan_keys: list | None = None
        self.graph_replays = 0
        self.prepared_replays = 0    # replays whose tables were made while the step before was still running

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
            logits = self._run_graph(rows) if self.use_graphs else None
            if logits is None:
                batch = self.builder.build(rows, self.model.spec.vocab)
        except Exception:
            for rid in new_requests:
                self.cache.free(rid)
            raise
        if logits is None:
            self.last_upload_bytes = batch.host_buffer.numel() * batch.host_buffer.element_size()
            self._zero_new_state(rows)
            logits = self.model.forward(batch, self.storage)
            if self._plan_keys is None:
                self._plan_keys = sorted(batch.attention_plans, key=repr)
        for (e, _, end) in plan:
            self.cache.commit(e.request_id, end)
        self.steps_run += 1
        return logits

    def _run_graph(self, rows):
        """Logits of a decode step through a captured graph, or None when the step is not one (or cannot be captured yet:
        the first steps of a model run eagerly and tell which attention plans its mixers ask for)."""
        if self._plan_keys is None or not all(len(r[2]) == 1 and list(r[3]) == [0] for r in rows):
            return None
        ht = self.builder.host_tables(rows, self.model.spec.vocab)
        kv_cap = -(-ht.max_kv_len // GRAPH_KV_GRANULE) * GRAPH_KV_GRANULE
        key = (ht.num_rows, kv_cap)
        g = self._graphs.get(key)
        if g is None:
            if len(self._graphs) >= MAX_GRAPHS:
                self._graphs.pop(next(iter(self._graphs)))
            g = self._graphs[key] = DecodeGraph(self, ht.num_rows, kv_cap, self._plan_keys)
        if not g.fits(ht):
            return None
        self.last_upload_bytes = g.static.total * 4
        self.graph_replays += 1
        return g.run(ht)

    # ------------------------------------------------------------------ a decode step prepared ahead of its tokens
    def prepare_decode(self, request_ids: list) -> PreparedDecode | None:
        """Everything of the next decode step of these requests (one token each, logits wanted) that does not depend on
        the tokens' values: pages, tables, attention work lists. A caller makes it while the device still runs the step
        before, and hands it to ``run_prepared`` with the tokens once they are known; when the next step turns out to be
        another one, the preparation is simply dropped (the pages it took belong to their requests and go back with
        them). None when the step cannot be prepared: no captured graph serves it yet, or pages are short."""
        if not self.use_graphs or self._plan_keys is None or not request_ids:
            return None
        max_pos = self.model.spec.max_positions
        need = [0] * len(self.groups)
        starts = []
        for rid in request_ids:
            if rid not in self.cache:
                return None
            start = self.cache.get(rid).tokens
            if max_pos and start + 1 > max_pos:
                return None
            starts.append(start)
            for gi, n in enumerate(self.cache.pages_needed(rid, start + 1)):
                need[gi] += n
        if any(n > self.cache.pools[gi].free_count for gi, n in enumerate(need)):
            return None
        rows = [(self.cache.extend(rid, start + 1), start, [0], [0]) for rid, start in zip(request_ids, starts)]
        ht = self.builder.host_tables(rows, self.model.spec.vocab)
        kv_cap = -(-ht.max_kv_len // GRAPH_KV_GRANULE) * GRAPH_KV_GRANULE
        g = self._graphs.get((ht.num_rows, kv_cap))
        if g is None or g.graph is None or not g.fits(ht):
            return None
        return PreparedDecode(list(request_ids), starts, g, g.static.stage(g._pending, g.fills))

    def matches_prepared(self, prep: PreparedDecode, entries: list[StepEntry]) -> bool:
        return (len(entries) == len(prep.request_ids) and prep.graph.graph is not None
                and self._graphs.get((prep.graph.num_rows, prep.graph.kv_cap)) is prep.graph
                and all(e.request_id == rid and len(e.tokens) == 1 and list(e.want) == [0] and (e.start is None or e.start == st)
                        and rid in self.cache and self.cache.get(rid).tokens == st
                        for e, rid, st in zip(entries, prep.request_ids, prep.starts)))

    def run_prepared(self, prep: PreparedDecode, entries: list[StepEntry]) -> torch.Tensor:
        """The step ``prepare_decode`` prepared, with its tokens. Call only when ``matches_prepared`` holds."""
        vocab = self.model.spec.vocab
        ids = prep.graph.static.staged(prep.staged, 0)
        for i, e in enumerate(entries):
            t = int(e.tokens[0])
            if not 0 <= t < vocab:
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab}")
            ids[i] = t
        logits = prep.graph.run_staged(prep.staged)
        self.last_upload_bytes = prep.graph.static.total * 4
        self.graph_replays += 1
        self.prepared_replays += 1
        for rid, st in zip(prep.request_ids, prep.starts):
            self.cache.commit(rid, st + 1)
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

    def close(self) -> None:
        """Drops the captured graphs and the cache's device memory."""
        self._graphs.clear()
        self.cache.free_all()
        self.storage.tensors.clear()
        self.storage._view_of_run.clear()

    def finish(self, request_id) -> None:
        """The request is done: everything it holds goes back to the pools."""
        self.cache.free(request_id)

    def tokens_cached(self, request_id) -> int:
        return self.cache.get(request_id).tokens if request_id in self.cache else 0
