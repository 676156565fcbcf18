"""The tables of one step, built on the host and copied to the device in one transfer.

A step is a list of rows; each row is one request's next tokens at consecutive positions: a whole prompt, a
portion of one, or a single decoded token, mixed freely. From the rows and the requests' block tables the
tables below are derived, the same set the reference's worker fills before every forward pass
(src/Starlings.Roost.Worker/Eager/PlanRegionWriter.cs:19-64): token ids, absolute positions, the slot each
token's key and value go to, per-row query and page ranges, the rows whose logits are wanted.

Two placements: a fresh pinned buffer and device buffer per step (any step), or a ``StaticTables`` of fixed
capacity whose device addresses never change, which a captured CUDA graph of a decode step reads on every replay.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.block_pool import NULL_PAGE


def pad_row(tokens: int) -> tuple:
    """A row that only fills a captured step up to the rows and tokens it was captured for: ``tokens`` tokens (id 0,
    possibly none) at position -1 of no request. It holds no keys (kv_len 0, an empty page range), writes no key or
    value (slot -1, which the cache write skips), gets no work from any mixer and wants no logits. A token's values never
    mix with another row's, so whatever a padding row carries stays in it."""
    return (None, -1, [0] * tokens, [])


def padded_rows(rows: list, tokens_cap: int, rows_cap: int) -> list:
    """``rows`` followed by padding rows, up to ``rows_cap`` rows and ``tokens_cap`` tokens: the padding tokens go
    one to a padding row, what is left over to the first of them."""
    pad_rows = rows_cap - len(rows)
    pad_tokens = tokens_cap - sum(len(r[2]) for r in rows)
    if pad_rows < 0 or pad_tokens < 0 or (pad_tokens and not pad_rows):
        raise ValueError(f"{len(rows)} rows do not fit a step of {rows_cap} rows and {tokens_cap} tokens")
    out = list(rows)
    for i in range(pad_rows):
        n = min(1, pad_tokens) if i else pad_tokens - min(pad_tokens, pad_rows - 1)
        out.append(pad_row(n))
        pad_tokens -= n
    return out


@dataclass
class GroupTables:
    """Per cache group. Paged: ``slot_mapping[t]`` = page * page_size + offset for token t, ``kv_indices``
    the rows' block tables back to back (a page given back to the pool stays as -1), ``kv_indptr`` their
    bounds. State: ``state_slots[b]`` the row's slot (a padding row names the group's scratch slot, which belongs to no
    request), ``fresh[b]`` 1 when the row brings its request's first token: the slot is zeroed before the step's blocks
    run."""
    slot_mapping: torch.Tensor | None = None
    kv_indptr: torch.Tensor | None = None
    kv_indices: torch.Tensor | None = None
    state_slots: torch.Tensor | None = None
    fresh: torch.Tensor | None = None


def upload_tables(arrays: list, device) -> tuple[list, torch.Tensor | None]:
    """int32 arrays in one pinned buffer (each starting on a 16-byte boundary), copied to the device in one transfer;
    (one device tensor per array, the pinned buffer, to be kept until the copy has run)."""
    offsets, total = [], 0
    for a in arrays:
        offsets.append(total)
        total += -(-a.size // 4) * 4
    if total == 0:
        return [None] * len(arrays), None
    device = torch.device(device)
    host = torch.zeros(total, dtype=torch.int32, pin_memory=device.type == "cuda")
    hv = host.numpy()
    for a, o in zip(arrays, offsets):
        hv[o : o + a.size] = a
    dev = host.to(device, non_blocking=True)
    return [dev[o : o + a.size] if a.size else None for a, o in zip(arrays, offsets)], host


def graph_kv_cap(kv_len: int) -> int:
    """The bound on the requests' lengths a captured decode step is made for: the next multiple of 1024 up to 8192
    tokens, of 4096 up to 32768, of 16384 beyond. It sizes the step's page tables and the mixers' work lists, whose unused
    entries cost an upload of a few bytes each and nothing on the device."""
    for limit, granule in ((8192, 1024), (32768, 4096)):
        if kv_len <= limit:
            return max(granule, -(-kv_len // granule) * granule)
    return -(-kv_len // 16384) * 16384


ROTATION_TABLE_MIN_TOKENS = 64   # from this many tokens on a step computes its cosines and sines once for all layers


@dataclass
class StepBatch:
    num_tokens: int
    num_rows: int
    num_selected: int
    ids: torch.Tensor            # [T] int32
    positions: torch.Tensor      # [T] int32 absolute position of each token
    token_row: torch.Tensor      # [T] int32 row of each token
    q_indptr: torch.Tensor       # [B+1] int32 token range of each row
    kv_lens: torch.Tensor        # [B] int32 tokens of the row's request once this step has run
    selected: torch.Tensor       # [S] int32 token indices whose logits are wanted
    groups: list = field(default_factory=list)
    # host-side facts, for parts written in Python and for kernel selection
    row_starts: list = field(default_factory=list)       # first position of each row
    row_counts: list = field(default_factory=list)       # tokens of each row
    max_position: int = 0
    max_kv_len: int = 0
    kv_cap: int = 0              # the bound on the requests' lengths a captured step of this size is made for
    all_single: bool = False     # every row brings exactly one token
    host_buffer: object = None   # the pinned staging buffer, kept until the step is done
    # key -> (the mixer that made it, what it bound): per-step work lists of mixers whose kernels want them, made by the
    # first run that asks and shared by every run that asks under the same key (see ``Mixer.step_work_arrays``)
    work: dict = field(default_factory=dict)
    rotation_tables: dict = field(default_factory=dict)   # frequency table -> the step's cosines and sines, made by the first layer that asks

    def rotation_table(self, kernels, inv_freq: torch.Tensor):
        """The cosines and sines of this step's positions for the frequencies ``inv_freq`` (float32 [T, half, 2]): they
        are the same in every layer, so the first layer that asks computes them and the others read them. None when
        the kernel library has no such entry point, and for steps of few tokens: there a layer's kernel computes its
        angles while its loads are in flight, and reading a table instead was measured slower (4.58 against 4.51 ms a
        decode step at the 8B sizes; a 2048-token prefill gains 0.7 ms)."""
        make = getattr(kernels, "rope_table", None)
        if make is None or inv_freq is None or self.num_tokens < ROTATION_TABLE_MIN_TOKENS:
            return None
        key = (inv_freq.data_ptr(), inv_freq.numel())
        table = self.rotation_tables.get(key)
        if table is None:
            table = self.rotation_tables[key] = make(self.positions, inv_freq)
        return table

    def step_work(self, mixer, key):
        """What ``mixer`` bound for this step under ``key``: its work lists, derived on the host from the rows' starts
        and counts, uploaded in one copy and bound by ``mixer.step_work_bind``. In a captured step the lists are there
        already, at fixed addresses (the executor's ``StepGraph`` refills them before every replay)."""
        entry = self.work.get(key)
        if entry is None:
            arrays = mixer.step_work_arrays(key, self.row_starts, self.row_counts)
            tensors, host = upload_tables(arrays, self.ids.device)
            bound = mixer.step_work_bind(key, tensors, host_arrays=arrays)
            entry = self.work[key] = (mixer, bound, host)
        return entry[1]


@dataclass
class HostTables:
    """A step's tables as numpy arrays, in placement order, with the facts a StepBatch carries on the host."""
    arrays: list
    num_tokens: int
    num_rows: int
    num_selected: int
    row_starts: list
    row_counts: list
    max_position: int
    max_kv_len: int


class StaticTables:
    """Device memory of fixed capacity for a step's tables, with a ring of pinned host buffers. The device addresses
    of all sections stay the same from step to step, so a captured graph can read them on every replay."""

    RING = 4

    def __init__(self, device, caps: list[int]):
        self.device = torch.device(device)
        self.caps = list(caps)
        self.offsets, total = [], 0
        for c in self.caps:
            self.offsets.append(total)
            total += -(-max(c, 1) // 4) * 4
        self.total = total
        self.dev = torch.zeros(total, dtype=torch.int32, device=self.device)
        self.hosts = [torch.zeros(total, dtype=torch.int32, pin_memory=self.device.type == "cuda") for _ in range(self.RING)]
        self.events = [None] * self.RING
        self.turn = 0
        self.views = [self.dev[o : o + max(c, 1)] for o, c in zip(self.offsets, self.caps)]

    def fits(self, arrays: list) -> bool:
        return len(arrays) == len(self.caps) and all(a.size <= c for a, c in zip(arrays, self.caps))

    def stage(self, arrays: list, fills: list) -> int:
        """Writes the arrays into the next pinned buffer (the rest of each section filled with ``fills[i]``) and returns
        its index; ``send`` copies it to the device. Between the two the caller may still change values in place
        through ``staged``."""
        i = self.turn
        self.turn = (self.turn + 1) % self.RING
        if self.events[i] is not None:
            self.events[i].synchronize()  # the copy that last read this host buffer is done
        hv = self.hosts[i].numpy()
        for a, o, c, f in zip(arrays, self.offsets, self.caps, fills):
            hv[o : o + a.size] = a
            hv[o + a.size : o + c] = f
        return i

    def staged(self, i: int, section: int):
        """The pinned copy of one section, as a numpy view."""
        o = self.offsets[section]
        return self.hosts[i].numpy()[o : o + self.caps[section]]

    def send(self, i: int) -> None:
        self.dev.copy_(self.hosts[i], non_blocking=True)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self.events[i] = ev

    def upload(self, arrays: list, fills: list) -> None:
        """Copies the arrays into their sections; the rest of each section is filled with ``fills[i]``."""
        self.send(self.stage(arrays, fills))


class BatchBuilder:
    """Derives a step's tables and places them: a fresh pinned buffer copied to the device once, or a StaticTables."""

    def __init__(self, device, cache_manager):
        self.device = torch.device(device)
        self.cm = cache_manager

    def host_tables(self, rows: list[tuple], vocab: int) -> HostTables:
        """rows: (request cache, start position, token list, wanted offsets within the tokens)."""
        T = sum(len(r[2]) for r in rows)
        B = len(rows)
        ids = np.empty(T, np.int32)
        pos = np.empty(T, np.int32)
        trow = np.empty(T, np.int32)
        q_indptr = np.zeros(B + 1, np.int32)
        kv_lens = np.empty(B, np.int32)
        selected = []
        at = 0
        for b, (rc, start, tokens, want) in enumerate(rows):
            n = len(tokens)
            ids[at : at + n] = tokens
            pos[at : at + n] = np.arange(start, start + n, dtype=np.int32) if rc is not None else -1
            trow[at : at + n] = b
            q_indptr[b + 1] = at + n
            kv_lens[b] = start + n if rc is not None else 0
            selected.extend(at + w for w in want)
            at += n
        if T and (ids.min() < 0 or ids.max() >= vocab):
            bad = int(ids[(ids < 0) | (ids >= vocab)][0])
            raise ValueError(f"token id {bad} is outside the vocabulary of {vocab}")
        arrays = [ids, pos, trow, q_indptr, kv_lens, np.asarray(selected, np.int32)]
        for gi, g in enumerate(self.cm.groups):
            if g.kind == "paged":
                slot = np.empty(T, np.int32)
                indptr = np.zeros(B + 1, np.int32)
                indices = []
                at = 0
                for b, (rc, start, tokens, _) in enumerate(rows):
                    n = len(tokens)
                    if rc is None:     # padding: nothing is written, no pages are read
                        slot[at : at + n] = -1
                        indptr[b + 1] = len(indices)
                        at += n
                        continue
                    table = rc.tables[gi]
                    if n == 1:
                        page = table[start // g.page_size]
                        if page == NULL_PAGE:
                            raise RuntimeError(f"request {rc.request_id!r}: a token of this step falls in a page that was given back")
                        slot[at] = page * g.page_size + start % g.page_size
                    else:
                        p = np.arange(start, start + n)
                        pages = np.asarray(table, np.int64)[p // g.page_size]
                        if (pages == NULL_PAGE).any():
                            raise RuntimeError(f"request {rc.request_id!r}: a token of this step falls in a page that was given back")
                        slot[at : at + n] = pages * g.page_size + p % g.page_size
                    used = -(-(start + n) // g.page_size)
                    indices.extend(table[:used])
                    indptr[b + 1] = len(indices)
                    at += n
                arrays += [slot, indptr, np.asarray(indices, np.int32)]
            else:
                scratch = self.cm.pools[gi].capacity       # the slot beyond the pool's: padding rows' state goes there
                arrays.append(np.asarray([rc.slots[gi] if rc is not None else scratch for rc, *_ in rows], np.int32))
                arrays.append(np.asarray([1 if rc is not None and start == 0 else 0 for rc, start, *_ in rows], np.int32))
        return HostTables(arrays=arrays, num_tokens=T, num_rows=B, num_selected=len(selected), row_starts=[r[1] for r in rows],
                          row_counts=[len(r[2]) for r in rows], max_position=max(int(pos.max()), 0) if T else 0,
                          max_kv_len=int(kv_lens.max()) if B else 0)

    def _batch(self, ht: HostTables, views: list, host_buffer) -> StepBatch:
        d_ids, d_pos, d_trow, d_qi, d_kvl, d_sel = views[:6]
        rest = views[6:]
        groups = []
        for g in self.cm.groups:
            if g.kind == "paged":
                groups.append(GroupTables(slot_mapping=rest[0], kv_indptr=rest[1], kv_indices=rest[2]))
                rest = rest[3:]
            else:
                groups.append(GroupTables(state_slots=rest[0], fresh=rest[1]))
                rest = rest[2:]
        return StepBatch(num_tokens=ht.num_tokens, num_rows=ht.num_rows, num_selected=ht.num_selected, ids=d_ids, positions=d_pos,
                         token_row=d_trow, q_indptr=d_qi, kv_lens=d_kvl, selected=d_sel, groups=groups, row_starts=ht.row_starts,
                         row_counts=ht.row_counts, max_position=ht.max_position, max_kv_len=ht.max_kv_len,
                         kv_cap=graph_kv_cap(ht.max_kv_len), all_single=all(n == 1 for n in ht.row_counts), host_buffer=host_buffer)

    def build(self, rows: list[tuple], vocab: int) -> StepBatch:
        return self.place(self.host_tables(rows, vocab))

    def place(self, ht: HostTables) -> StepBatch:
        """The tables in a fresh pinned buffer, copied to the device in one transfer."""
        flat = ht.arrays
        offsets, total = [], 0
        for a in flat:  # 16-byte aligned sub-tables in one buffer
            offsets.append(total)
            total += -(-a.size // 4) * 4
        host = torch.empty(max(total, 4), dtype=torch.int32, pin_memory=self.device.type == "cuda")
        hv = host.numpy()
        for a, o in zip(flat, offsets):
            hv[o : o + a.size] = a
        dev = host.to(self.device, non_blocking=True)
        views = [dev[o : o + a.size] for a, o in zip(flat, offsets)]
        return self._batch(ht, views, host)

    # ------------------------------------------------------------------ fixed placement for graph replay
    def table_caps(self, num_tokens: int, num_rows: int, kv_cap: int) -> list[int]:
        """Capacities, in placement order, of the tables of a step of ``num_tokens`` tokens in ``num_rows`` rows whose
        requests hold at most ``kv_cap`` tokens and which wants at most one row of logits a row."""
        T, B = num_tokens, num_rows
        caps = [T, T, T, B + 1, B, B]
        for g in self.cm.groups:
            if g.kind == "paged":
                caps += [T, B + 1, B * (-(-kv_cap // g.page_size))]
            else:
                caps += [B, B]
        return caps

    def static_batch(self, ht: HostTables, static: StaticTables, n_table_sections: int) -> StepBatch:
        """A batch over the fixed tables, with the counts of the step they were made for (``ht`` filled up with padding
        rows): every table at its capacity, as many logits as rows."""
        full = HostTables(arrays=ht.arrays, num_tokens=ht.num_tokens, num_rows=ht.num_rows, num_selected=ht.num_rows,
                          row_starts=ht.row_starts, row_counts=ht.row_counts, max_position=ht.max_position, max_kv_len=ht.max_kv_len)
        return self._batch(full, static.views[:n_table_sections], None)
