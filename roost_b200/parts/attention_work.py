"""The work lists of the tensor-core attention kernels: how a step's rows are divided among them.

The paged-attention mixer owns these lists. It hands them to the step's batch as its per-step work (``Mixer.step_work_*``
in ``parts/base.py``): the batch builds them once a step for all the layers that share a geometry, and a captured step
keeps them at fixed device addresses and refills them on every replay, without either knowing what the lists hold.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


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
    cluster_chunks: int = 0      # > 0: the decode list holds this many items a row, for clusters of as many CTAs (no merge list)
    prefill_work: torch.Tensor | None = None
    decode_work: torch.Tensor | None = None
    merge_work: torch.Tensor | None = None


def attention_work(row_starts, row_counts, group: int, window: int | None, chunk: int, tile_rows: int = 64, cluster: int = 0):
    """(prefill pairs, decode quadruples, merge quadruples, slots) as flat int lists. ``chunk`` is a multiple of 64: a
    chunk starts on a boundary of the decode kernels' key tiles. With ``cluster`` = S > 0 a short row gets exactly S
    decode items (its chunks in key order, then empty ones) for a cluster of S CTAs that merges them itself: no merge
    items and no slots."""
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
            if cluster:
                if len(begins) > cluster:
                    raise ValueError(f"a row of {kv_len} keys has {len(begins)} chunks of {chunk}: more than the cluster's {cluster}")
                for r in range(cluster):
                    c = first + r * chunk
                    decode += [b, c, min(c + chunk, kv_len), r] if c < kv_len else [b, 0, 0, r]
            elif len(begins) == 1:
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
                   short_rows: bool = True, cluster: int = 0) -> tuple[int, int, int]:
    """Largest (prefill, decode, merge) item counts of a step of ``num_tokens`` tokens in ``num_rows`` rows whose
    requests hold at most ``kv_cap`` keys. A step of one token a row has work of one kind only; so has a step without
    ``short_rows`` (rows of at most 16 tokens, the only ones that can go to the decode kernel)."""
    chunks = cluster if cluster else -(-kv_cap // chunk)
    merges = 0 if cluster else num_rows
    if num_tokens == num_rows:
        if group > 16:
            return num_rows * (-(-group // tile_rows)), 0, 0
        return 0, num_rows * chunks, merges
    prefill = -(-num_tokens * group // tile_rows) + num_rows
    return (prefill, num_rows * chunks, merges) if short_rows else (prefill, 0, 0)


def _pad4(a: list) -> list:
    return a + [0] * (-len(a) % 4)


def plan_attention(row_starts, row_counts, group: int, window: int | None, chunk: int, device, tile_rows: int = 64,
                   cluster: int = 0) -> AttentionPlan:
    """The lists of one step on the device, for callers that run the attention kernels outside an engine (kernel tests,
    microbenchmarks)."""
    prefill, decode, merge, slots = attention_work(row_starts, row_counts, group, window, chunk, tile_rows, cluster)
    plan = AttentionPlan(prefill_items=len(prefill) // 2, prefill_tile_rows=tile_rows, decode_items=len(decode) // 4, merge_items=len(merge) // 4, slots=slots,
                         merge_rows=max((z >> 24 for z in merge[2::4]), default=1), cluster_chunks=cluster)
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
