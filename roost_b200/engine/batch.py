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
    value (slot -1, which the cache write skips), gets no attention work and wants no logits. A token's values never
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
    bounds. State: ``state_slots[b]`` the row's slot."""
    slot_mapping: torch.Tensor | None = None
    kv_indptr: torch.Tensor | None = None
    kv_indices: torch.Tensor | None = None
    state_slots: torch.Tensor | None = None


@dataclass
class AttentionPlan:
    """How the tensor-core attention kernels divide a step's rows (see csrc/attention_mma.cu): rows with at most 16
    packed rows (tokens x query heads per key/value head) go to the decode kernel in chunks of a fixed number of
    keys, the others to the prefill kernel in tiles of ``prefill_tile_rows`` packed rows. Item counts may include
    padding entries (batch row -1), which the kernels skip."""
    prefill_items: int = 0
    prefill_tile_rows: int = 64
    merge_rows: int = 16         # the most packed rows a split row has (the merge kernel's blocks along z)
    decode_items: int = 0
    merge_items: int = 0
    slots: int = 0
    prefill_work: torch.Tensor | None = None
    decode_work: torch.Tensor | None = None
    merge_work: torch.Tensor | None = None


def attention_work(row_starts, row_counts, group: int, window: int | None, chunk: int, tile_rows: int = 64):
    """(prefill pairs, decode quadruples, merge quadruples, slots) as flat int lists. ``chunk`` is a multiple of 64: a
    chunk starts on a boundary of the decode kernels' key tiles."""
    if chunk <= 0 or chunk % 64:
        raise ValueError(f"decode chunk {chunk} is not a positive multiple of 64")
    prefill, decode, merge, tiles = [], [], [], []
    slots = 0
    token = 0    # the row's first token among the step's tokens
    for b, (start, n) in enumerate(zip(row_starts, row_counts)):
        rows, kv_len = n * group, start + n
        first_token, token = token, token + n
        if start < 0:
            continue   # a padding row (see pad_row): no keys, no work
        if rows <= 16:
            lo = max(0, start - window + 1) if window else 0
            first = (lo // chunk) * chunk
            begins = range(first, kv_len, chunk)
            if len(begins) == 1:
                decode += [b, first, min(first + chunk, kv_len), -1]
            else:
                merge += [b, slots, len(begins) | (rows << 24), first_token]
                for c in begins:
                    decode += [b, c, min(c + chunk, kv_len), slots]
                    slots += 1
        else:
            for r0 in range(0, rows, tile_rows):
                tiles.append((start + min(rows, r0 + tile_rows) // group, b, r0))
    # the tiles with the longest history run longest: they go first, so that the last wave of CTAs is the lightest
    for _, b, r0 in sorted(tiles, key=lambda t: -t[0]):
        prefill += [b, r0]
    return prefill, decode, merge, slots


def attention_caps(num_tokens: int, num_rows: int, kv_cap: int, group: int, chunk: int, tile_rows: int = 64,
                   short_rows: bool = True) -> tuple[int, int, int]:
    """Largest (prefill, decode, merge) item counts of a step of ``num_tokens`` tokens in ``num_rows`` rows whose
    requests hold at most ``kv_cap`` keys. A step of one token a row has work of one kind only; so has a step without
    ``short_rows`` (rows of at most 16 tokens, the only ones that can go to the decode kernel)."""
    chunks = -(-kv_cap // chunk)
    if num_tokens == num_rows:
        if group > 16:
            return num_rows * (-(-group // tile_rows)), 0, 0
        return 0, num_rows * chunks, num_rows
    prefill = -(-num_tokens * group // tile_rows) + num_rows
    return (prefill, num_rows * chunks, num_rows) if short_rows else (prefill, 0, 0)


def _pad4(a: list) -> list:
    return a + [0] * (-len(a) % 4)


def plan_attention(row_starts, row_counts, group: int, window: int | None, chunk: int, device, tile_rows: int = 64) -> AttentionPlan:
    prefill, decode, merge, slots = attention_work(row_starts, row_counts, group, window, chunk, tile_rows)
    plan = AttentionPlan(prefill_items=len(prefill) // 2, prefill_tile_rows=tile_rows, decode_items=len(decode) // 4, merge_items=len(merge) // 4, slots=slots,
                         merge_rows=max((z >> 24 for z in merge[2::4]), default=1))
    flat = _pad4(prefill) + _pad4(decode) + _pad4(merge)
    if flat:
        host = torch.tensor(flat, dtype=torch.int32)
        if torch.device(device).type == "cuda":
            host = host.pin_memory()
        dev = host.to(device, non_blocking=True)
        a = len(_pad4(prefill))
        b_ = a + len(_pad4(decode))
        plan.prefill_work, plan.decode_work, plan.merge_work = dev[:a], dev[a:b_], dev[b_:]
        plan.host = host
    return plan


def graph_kv_cap(kv_len: int) -> int:
    """The bound on the requests' lengths a captured decode step is made for: the next multiple of 1024 up to 8192
    tokens, of 4096 up to 32768, of 16384 beyond. It sizes the step's page tables and attention work lists, whose unused
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
    attention_plans: dict = field(default_factory=dict)   # (group size, window, chunk) -> AttentionPlan, made by the first mixer that asks
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

    def attention_plan(self, group: int, window: int | None, chunk: int, tile_rows: int = 64) -> AttentionPlan:
        key = (group, window, chunk, tile_rows)
        plan = self.attention_plans.get(key)
        if plan is None:
            plan = plan_attention(self.row_starts, self.row_counts, group, window, chunk, self.ids.device, tile_rows)
            self.attention_plans[key] = plan
        return plan


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
                arrays.append(np.asarray([rc.slots[gi] if rc is not None else 0 for rc, *_ in rows], np.int32))
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
                groups.append(GroupTables(state_slots=rest[0]))
                rest = rest[1:]
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
                caps.append(B)
        return caps

    def static_batch(self, ht: HostTables, static: StaticTables, n_table_sections: int) -> StepBatch:
        """A batch over the fixed tables, with the counts of the step they were made for (``ht`` filled up with padding
        rows): every table at its capacity, as many logits as rows."""
        full = HostTables(arrays=ht.arrays, num_tokens=ht.num_tokens, num_rows=ht.num_rows, num_selected=ht.num_rows,
                          row_starts=ht.row_starts, row_counts=ht.row_counts, max_position=ht.max_position, max_kv_len=ht.max_kv_len)
        return self._batch(full, static.views[:n_table_sections], None)
