"""Grouped-query causal attention over the paged cache, as a mixer.

Per step: one fused qkv projection; one kernel that norms the q and k heads, rotates them and writes k and v
into the step's page slots; attention of the step's queries over the pages (the keys this step wrote
included); the output projection. The order of operations is the reference's node list for the dense Qwen3
layer (src/Starlings.Roost.Models.Tiny/RoostTiny.cs:41-48): projections, QkNorm, Rope, CacheWrite,
PagedAttention, o_proj. The qkv rows hold [q heads | k heads | v heads], the row layout of the reference's
fused op (src/Starlings.Roost.Ops/CpuOps.Fused.cs:39-41).
"""
from __future__ import annotations

import torch

import numpy as np

from ..config.spec import AttentionSpec
from .attention_work import AttentionPlan, attention_caps, attention_work
from .base import NORMS, POSITIONS, CacheNeed, Mixer, ParamDecl, Runtime, register_mixer
from .linear import Linear

SHORT_ROW_TOKENS = 16   # rows of at most this many tokens may go to the split decode kernel


class PagedAttention(Mixer):
    def __init__(self, spec: AttentionSpec, runtime: Runtime):
        s = spec
        if min(s.hidden, s.num_heads, s.num_kv_heads, s.head_dim) <= 0:
            raise ValueError("paged_attention: hidden, head counts and head_dim must be positive")
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"paged_attention: {s.num_heads} query heads are not a multiple of {s.num_kv_heads} key/value heads")
        if s.head_dim % 2:
            raise ValueError(f"paged_attention: head_dim {s.head_dim} is odd")
        if s.head_dim > 512:
            raise ValueError(f"paged_attention: head_dim {s.head_dim} is beyond 512, the largest any kernel here serves")
        if s.window is not None and s.window <= 0:
            raise ValueError(f"paged_attention: window {s.window} must be positive")
        if s.scale <= 0:
            raise ValueError(f"paged_attention: scale {s.scale} must be positive")
        self.spec = s
        self.rt = runtime
        self.q_width = s.num_heads * s.head_dim
        self.kv_width = s.num_kv_heads * s.head_dim
        self.qkv = Linear(runtime, self.q_width + 2 * self.kv_width, s.hidden)
        self.out = Linear(runtime, s.hidden, self.q_width)
        self.q_only: Linear | None = None   # the q rows of qkv, for runs that read another run's cache
        self.q_norm = self.k_norm = None
        if s.qk_norm is not None:
            if s.qk_norm.size != s.head_dim:
                raise ValueError("paged_attention: the q/k norm must span head_dim")
            self.q_norm = NORMS.build(s.qk_norm, runtime)
            self.k_norm = NORMS.build(s.qk_norm, runtime)
        self.position = POSITIONS.build(s.position, runtime) if s.position is not None else None

    @classmethod
    def parameters(cls, spec: AttentionSpec):
        Q, KV, H, d = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim, spec.hidden, spec.head_dim
        p = {"qkv": ParamDecl(shape=(Q + 2 * KV, H), row_splits=(Q, KV, KV)), "out": ParamDecl(shape=(H, Q))}
        if spec.qk_norm is not None:
            p["q_norm"] = ParamDecl(shape=(d,), role="vector")
            p["k_norm"] = ParamDecl(shape=(d,), role="vector")
        return p

    def load(self, params):
        self.qkv.load(params["qkv"])
        self.out.load(params["out"])
        if self.q_norm is not None:
            self.q_norm.load({"weight": params["q_norm"]})
            self.k_norm.load({"weight": params["k_norm"]})

    def cache_need(self) -> CacheNeed:
        s = self.spec
        return CacheNeed(kind="paged", kv_heads=s.num_kv_heads, head_dim=s.head_dim, window=s.window)

    def __call__(self, x, batch, cache, write_cache: bool = True):
        s, k = self.spec, self.rt.kernels
        tables = batch.groups[cache.group]
        inv_freq, rotary_dim = self.position.rotation() if self.position is not None else (None, 0)
        if self.position is not None and self.position.max_positions and batch.max_position >= self.position.max_positions:
            raise ValueError(f"position {batch.max_position} is beyond the model's {self.position.max_positions} positions")
        eps = s.qk_norm.eps if s.qk_norm is not None else 1.0
        qw = self.q_norm.weight if self.q_norm is not None else None
        kw = self.k_norm.weight if self.k_norm is not None else None
        own_table = getattr(self.position, "step_table", None) if rotary_dim else None
        table = own_table(batch) if own_table is not None else None     # an encoding with angles of its own
        if table is None and rotary_dim:
            table = batch.rotation_table(k, inv_freq)
        if write_cache:
            qkv = self.qkv(x)
            q = k.qk_norm_rope_cache(qkv, s.num_heads, s.num_kv_heads, s.head_dim, q_w=qw, k_w=kw, eps=eps,
                                     inv_freq=inv_freq, rotary_dim=rotary_dim, positions=batch.positions, cos_sin=table,
                                     k_pool=cache.k_pool, v_pool=cache.v_pool, slot_mapping=tables.slot_mapping,
                                     page_size=cache.page_size, write_kv=True)
        else:
            if self.q_only is None:
                self.q_only = Linear(self.rt, self.q_width, s.hidden)
                self.q_only.load(self.qkv.weight[: self.q_width])
            q = k.qk_norm_rope_cache(self.q_only(x), s.num_heads, s.num_kv_heads, s.head_dim, q_w=qw, k_w=kw, eps=eps,
                                     inv_freq=inv_freq, rotary_dim=rotary_dim, positions=batch.positions, write_kv=False, cos_sin=table)
        o = self.attend(q, batch, cache, tables)
        return self.out(o)

    def attend(self, q, batch, cache, tables):
        """bfloat16 with a head size the tensor-core kernels serve goes to them; float32 and every other head size
        run the 32-bit kernel, which takes any size."""
        s, k = self.spec, self.rt.kernels
        if q.dtype == torch.bfloat16 and getattr(k, "attention_mma_supported", lambda d: False)(s.head_dim):
            group = s.num_heads // s.num_kv_heads
            tile_rows = k.attention_prefill_tile_rows(s.num_heads, cache.k_pool, cache.v_pool, batch.num_tokens * group)
            split_for = getattr(k, "decode_split_for", None)
            chunk, cluster = split_for(batch.num_rows, batch.kv_cap, cache.k_pool, cache.v_pool) if split_for and batch.kv_cap else (k.decode_chunk, 0)
            plan = batch.step_work(self, ("paged_attention", group, s.window, chunk, tile_rows, cluster))
            return k.attention_mma(q, cache.k_pool, cache.v_pool, batch.q_indptr, batch.kv_lens, tables.kv_indptr,
                                   tables.kv_indices, plan, s.scale, s.window)
        return k.paged_attention_generic(q, cache.k_pool, cache.v_pool, batch.positions, batch.token_row,
                                         tables.kv_indptr, tables.kv_indices, s.scale, s.window)


    # ---- the tensor-core kernels' work lists, as the step's batch asks for them
    def step_class(self, row_counts):
        return ("short_rows", any(n <= SHORT_ROW_TOKENS for n in row_counts))

    def step_work_arrays(self, key, row_starts, row_counts):
        _, group, window, chunk, tile_rows, cluster = key
        prefill, decode, merge, _ = attention_work(row_starts, row_counts, group, window, chunk, tile_rows, cluster)
        return [np.asarray(prefill, np.int32), np.asarray(decode, np.int32), np.asarray(merge, np.int32)]

    def step_work_caps(self, key, num_tokens, num_rows, kv_cap, step_class):
        _, group, _, chunk, tile_rows, cluster = key
        short = dict([step_class[i : i + 2] for i in range(0, len(step_class), 2)]).get("short_rows", True)
        pc, dc, mc = attention_caps(num_tokens, num_rows, kv_cap, group, chunk, tile_rows, short, cluster)
        return [(pc * 2, -1), (dc * 4, -1), (mc * 4, -1)]     # padding items name batch row -1, which the kernels skip

    def step_work_bind(self, key, tensors, host_arrays=None, captured=None):
        _, group, _, _, tile_rows, cluster = key
        prefill, decode, merge = tensors
        if captured is not None:       # every list at its capacity; a step of one token a row splits rows of `group` packed rows
            num_tokens, num_rows, kv_cap, step_class = captured
            (pc, _), (dc, _), (mc, _) = self.step_work_caps(key, num_tokens, num_rows, kv_cap, step_class)
            return AttentionPlan(prefill_items=pc // 2, prefill_tile_rows=tile_rows, decode_items=dc // 4, merge_items=mc // 4,
                                 slots=0 if cluster else dc // 4, cluster_chunks=cluster,
                                 merge_rows=min(16, group) if num_tokens == num_rows else 16, prefill_work=prefill, decode_work=decode,
                                 merge_work=merge)
        hp, hd, hm = host_arrays
        slots = 0 if cluster else int((hd[3::4] >= 0).sum())      # every chunk of a split row has a partial slot of its own
        return AttentionPlan(prefill_items=hp.size // 2, prefill_tile_rows=tile_rows, decode_items=hd.size // 4, merge_items=hm.size // 4,
                             slots=slots, cluster_chunks=cluster, merge_rows=int((hm[2::4] >> 24).max()) if hm.size else 1, prefill_work=prefill,
                             decode_work=decode, merge_work=merge)


register_mixer("paged_attention", PagedAttention)
