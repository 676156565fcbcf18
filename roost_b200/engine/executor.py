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
from .batch import BatchBuilder, HostTables, StaticTables, graph_kv_cap, padded_rows
from .model import Model

MAX_GRAPHS = 64
GRAPH_TOKENS = 2048   # a step of more tokens runs eagerly: the device bounds it, not the host's launches


def graph_tokens(n: int) -> int:
    """Tokens of the captured step that serves a step of ``n`` tokens of which some row brings more than one: 8, 16, 32,
    then the next multiple of 64 up to 512, of 128 up to 1024 and of 256 beyond. A scheduler that fills a token budget
    asks for the budget's own size step after step."""
    for m in (8, 16, 32):
        if n <= m:
            return m
    granule = 64 if n <= 512 else (128 if n <= 1024 else 256)
    return -(-n // granule) * granule


def graph_rows(n: int) -> int:
    """Rows of the captured decode step that serves ``n`` rows: up to 8 exactly, then 12, 16, 24, 32, 48, 64 and so on
    (at most half as many again), filled up with padding rows. A server's batch shrinks and grows by one request at a
    time; without the steps every size would be captured for itself."""
    if n <= 8:
        return n
    b = 8
    while True:
        for m in (b * 3 // 2, b * 2):
            if n <= m:
                return m
        b *= 2


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


class StepGraph:
    """A captured CUDA graph of one step for a fixed number of tokens and rows and a bound on the requests' lengths.
    The step's tables live at fixed device addresses; a replay uploads the new tables and launches the whole forward
    pass with one call, so the host's per-kernel launch cost (hundreds of launches a step) no longer bounds small
    batches and small models. A step with fewer rows or tokens is filled up with padding rows (``batch.pad_row``), the
    mixers' work lists with items their kernels skip. The reference's one graph experiment did not replay bit-identically
    and is unclaimed (kernels/README.md:240-250); here a replay runs the very kernels of the eager path with the same
    arguments, and the tests compare both with the plain implementation.

    ``work``: (key, mixer) of every set of per-step work lists the eager run of this step asked its batch for. The graph
    gives each list a fixed section beside the step's tables (sized by ``mixer.step_work_caps``), refills the sections
    from ``mixer.step_work_arrays`` before every replay and hands the mixer its sections once, at capture."""

    def __init__(self, executor: "StepExecutor", num_tokens: int, num_rows: int, kv_cap: int, step_class: tuple, work: list):
        self.ex = weakref.proxy(executor)   # the executor owns its graphs; no reference cycle keeps its cache alive
        self.num_tokens, self.num_rows, self.kv_cap, self.step_class = num_tokens, num_rows, kv_cap, step_class
        self.work = list(work)
        builder = executor.builder
        table_caps = builder.table_caps(num_tokens, num_rows, kv_cap)
        self.n_table = len(table_caps)
        caps, fills = list(table_caps), [0] * len(table_caps)
        self.work_sections = []             # per set of lists: the indices of its sections
        for key, mixer in self.work:
            sizes = mixer.step_work_caps(key, num_tokens, num_rows, kv_cap, step_class)
            self.work_sections.append(list(range(len(caps), len(caps) + len(sizes))))
            for cap, fill in sizes:
                caps.append(cap)
                fills.append(fill)
        self.fills = fills
        self.static = StaticTables(executor.rt.device, caps)
        self.graph = None
        self.out = None

    @property
    def key(self) -> tuple:
        return (self.num_tokens, self.num_rows, self.kv_cap, self.step_class)

    def _arrays(self, ht: HostTables) -> list:
        arrays = list(ht.arrays)
        for key, mixer in self.work:
            arrays += [np.asarray(a, np.int32) for a in mixer.step_work_arrays(key, ht.row_starts, ht.row_counts)]
        return arrays

    def fits(self, ht: HostTables) -> bool:
        self._pending = self._arrays(ht)
        return self.static.fits(self._pending)

    def run(self, live: int) -> torch.Tensor:
        """A replay with the tables of the last ``fits`` that returned True. ``live``: the rows of logits that are wanted."""
        self.static.upload(self._pending, self.fills)
        self.graph.replay()
        self._count()
        return self.out[:live].clone()

    def _count(self) -> None:
        k = self.ex.rt.kernels
        k.launches += self.launches
        k.library_launches = getattr(k, "library_launches", 0) + self.library_launches

    def run_staged(self, staged: int, live: int) -> torch.Tensor:
        """A replay with tables staged earlier."""
        self.static.send(staged)
        self.graph.replay()
        self._count()
        return self.out[:live].clone()

    def capture(self, ht: HostTables) -> None:
        """Records the step over the fixed tables (after ``fits(ht)`` returned True). Nothing runs: the step's own result
        comes from the eager run before it, which also told which work lists the model's mixers ask for."""
        ex = self.ex
        self.static.upload(self._pending, self.fills)
        batch = ex.builder.static_batch(ht, self.static, self.n_table)
        captured = (self.num_tokens, self.num_rows, self.kv_cap, self.step_class)
        for (key, mixer), sections in zip(self.work, self.work_sections):
            batch.work[key] = (mixer, mixer.step_work_bind(key, [self.static.views[i] for i in sections], captured=captured), None)
        graph = torch.cuda.CUDAGraph()
        before, before_lib = ex.rt.kernels.launches, getattr(ex.rt.kernels, "library_launches", 0)
        # one memory pool for all of an executor's graphs: they never run at the same time, so what one capture used
        # and freed serves the next
        with torch.cuda.graph(graph, pool=ex.graph_pool()):
            out = ex.forward(batch)
        self.launches = ex.rt.kernels.launches - before   # kernels of this library one replay launches
        self.library_launches = getattr(ex.rt.kernels, "library_launches", 0) - before_lib   # and cuBLAS products
        ex.rt.kernels.launches = before
        ex.rt.kernels.library_launches = before_lib
        if sorted(batch.work, key=repr) != sorted((k for k, _ in self.work), key=repr):
            raise RuntimeError("the captured step asked for other work lists than the eager step before it")
        self.graph, self.out, self.batch = graph, out, batch


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
        # steps are replayed from captured graphs when every part says that its call can be captured and every mixer
        # with state of its own says that it reads the step's device tables only (``Mixer.state_capturable``; a mixer
        # written in Python over host values is right as it is and keeps its model's steps eager)
        self.mixers = [b.mixer for b in model.blocks]
        state_runs = {r for g in self.groups if g.kind == "state" for r in g.runs}
        self.use_graphs = (use_graphs and self.rt.device.type == "cuda"
                           and all(getattr(model.blocks[model.spec.schedule[r].block].mixer, "state_capturable", False) for r in state_runs)
                           and all(getattr(p, "capturable", True) for p in model.parts()))
        self._graphs: dict = {}
        self._graph_pool = None
        self._seen: dict = {}        # sizes of steps of several tokens a row that ran eagerly, and how often
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
            logits = self.forward(batch)
        for (e, _, end) in plan:
            self.cache.commit(e.request_id, end)
        self.steps_run += 1
        return logits

    def _run_graph(self, rows):
        """Logits of the step through a captured graph, or None when it is to run eagerly: a step of many tokens, one
        that wants more rows of logits than it has rows, or a step of several tokens a row whose sizes are seen for the
        first time (a decode step is captured at once, any other when its sizes come again)."""
        tokens, wanted = sum(len(r[2]) for r in rows), sum(len(r[3]) for r in rows)
        decode = all(len(r[2]) == 1 and list(r[3]) == [0] for r in rows)
        if decode:
            tokens_cap = rows_cap = graph_rows(len(rows))
        else:
            if tokens > GRAPH_TOKENS:
                return None
            tokens_cap = graph_tokens(tokens)
            rows_cap = graph_rows(len(rows) + (1 if tokens_cap > tokens else 0))
            if wanted > rows_cap:
                return None
        ht = self.builder.host_tables(padded_rows(rows, tokens_cap, rows_cap), self.model.spec.vocab)
        # what the mixers say about the step's rows decides which of their kernels a step needs at all (a step without
        # short rows is captured without the kernel that serves them): it is part of the captured step's identity
        key = (tokens_cap, rows_cap, graph_kv_cap(ht.max_kv_len), self.step_class([len(r[2]) for r in rows]))
        g = self._touch(key)
        if g is None:
            if not decode:
                if len(self._seen) > 4096:
                    self._seen.clear()
                self._seen[key] = self._seen.get(key, 0) + 1
                if self._seen[key] < 2:
                    return None
            # the eager run of the padded step gives this step's result and tells which work lists the mixers ask
            # for; the capture that follows records the same launches over fixed tables without running them
            batch = self.builder.place(ht)
            self.last_upload_bytes = batch.host_buffer.numel() * batch.host_buffer.element_size()
            logits = self.forward(batch)
            g = StepGraph(self, tokens_cap, rows_cap, key[2], key[3], [(k, batch.work[k][0]) for k in sorted(batch.work, key=repr)])
            if g.fits(ht):
                g.capture(ht)
                if len(self._graphs) >= MAX_GRAPHS:
                    self._graphs.pop(next(iter(self._graphs)))
                self._graphs[key] = g
            return logits[:wanted]
        if not g.fits(ht):
            return None
        self.last_upload_bytes = g.static.total * 4
        self.graph_replays += 1
        return g.run(wanted)

    def step_class(self, row_counts: list) -> tuple:
        out = ()
        for m in self.mixers:
            c = m.step_class(row_counts) if hasattr(m, "step_class") else ()
            if c and c not in out:
                out += (c,)
        return tuple(x for c in out for x in c)

    def _touch(self, key):
        """The captured step of this key, marked as the most recently used (the least recently used one goes when there
        are too many)."""
        g = self._graphs.pop(key, None)
        if g is not None:
            self._graphs[key] = g
        return g

    def graph_pool(self):
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        return self._graph_pool

    # ------------------------------------------------------------------ a decode step prepared ahead of its tokens
    def prepare_decode(self, request_ids: list) -> PreparedDecode | None:
        """Everything of the next decode step of these requests (one token each, logits wanted) that does not depend on
        the tokens' values: pages, tables, the mixers' work lists. A caller makes it while the device still runs the step
        before, and hands it to ``run_prepared`` with the tokens once they are known; when the next step turns out to be
        another one, the preparation is simply dropped (the pages it took belong to their requests and go back with
        them). None when the step cannot be prepared: no captured graph serves it yet, or pages are short."""
        if not self.use_graphs or not request_ids:
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
        cap = graph_rows(len(rows))
        ht = self.builder.host_tables(padded_rows(rows, cap, cap), self.model.spec.vocab)
        g = self._touch((cap, cap, graph_kv_cap(ht.max_kv_len), self.step_class([1] * len(rows))))
        if g is None or not g.fits(ht):
            return None
        return PreparedDecode(list(request_ids), starts, g, g.static.stage(g._pending, g.fills))

    def matches_prepared(self, prep: PreparedDecode, entries: list[StepEntry]) -> bool:
        return (len(entries) == len(prep.request_ids)
                and self._graphs.get(prep.graph.key) is prep.graph
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
        logits = prep.graph.run_staged(prep.staged, len(entries))
        self.last_upload_bytes = prep.graph.static.total * 4
        self.graph_replays += 1
        self.prepared_replays += 1
        for rid, st in zip(prep.request_ids, prep.starts):
            self.cache.commit(rid, st + 1)
        self.steps_run += 1
        return logits

    def launch_prepared(self, prep: PreparedDecode, ids_device: torch.Tensor) -> torch.Tensor:
        """Starts the prepared step with its token ids still on the device: the ids the step before has sampled, one a
        row, in the rows' order. The tables go up, the ids are copied into their table on the device, the graph is
        replayed. The host has read nothing: the caller may start this step before it knows the tokens of the step
        before. Nothing is committed either; ``adopt_prepared`` does that once the caller knows which rows stand (a row
        whose request turns out to have ended with the token before is simply dropped: what it wrote lies in pages
        that go back to the pool, and later launches come after it on the stream)."""
        n = len(prep.request_ids)
        if ids_device.numel() != n or ids_device.dtype != torch.int32:
            raise ValueError("launch_prepared: one int32 token id a row is needed")
        g = prep.graph
        g.static.send(prep.staged)
        g.static.views[0][:n].copy_(ids_device)
        g.graph.replay()
        g._count()
        self.last_upload_bytes = g.static.total * 4
        return g.out[:n].clone()

    def adoptable(self, prep: PreparedDecode, entries: list[StepEntry]) -> list[int] | None:
        """The rows of a step started by ``launch_prepared`` that these entries name, when the entries are exactly such
        a step: the same requests or some of them, in the same order, one token each at the position the step was
        prepared for, its logits wanted. None otherwise."""
        where = {rid: i for i, rid in enumerate(prep.request_ids)}
        keep, last = [], -1
        for e in entries:
            i = where.get(e.request_id)
            if (i is None or i <= last or len(e.tokens) != 1 or list(e.want) != [0] or e.request_id not in self.cache
                    or self.cache.get(e.request_id).tokens != prep.starts[i] or (e.start is not None and e.start != prep.starts[i])):
                return None
            keep.append(i)
            last = i
        return keep or None

    def adopt_prepared(self, prep: PreparedDecode, keep: list[int]) -> None:
        """The step started by ``launch_prepared`` stands for the rows ``keep``: their requests now hold one token more."""
        for i in keep:
            self.cache.commit(prep.request_ids[i], prep.starts[i] + 1)
        self.graph_replays += 1
        self.prepared_replays += 1
        self.steps_run += 1

    def forward(self, batch) -> torch.Tensor:
        """The model's forward pass over a step's batch, after the fixed-size state of every request whose first token
        the step brings has been set to zero, as the reference's worker zeroes a recurrent slot at position 0
        (src/Starlings.Roost.Worker/Eager/EagerWorker.cs:214-230). The zeroing reads the step's device tables only
        (``state_slots``, ``fresh``), so it is part of a captured step like everything after it; a padding row names the
        group's scratch slot."""
        for gi, g in enumerate(self.groups):
            if g.kind != "state" or not g.runs:
                continue
            tables = batch.groups[gi]
            state = self.storage.tensors[gi]                        # [runs, slots + 1, *shape]
            slots = tables.state_slots.long()
            keep = (1 - tables.fresh).to(state.dtype).view(1, -1, *([1] * (state.dim() - 2)))
            state.index_copy_(1, slots, state.index_select(1, slots) * keep)
        return self.model.forward(batch, self.storage)

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
