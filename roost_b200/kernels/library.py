"""The Python side of the kernel library's C ABI: loads the shared object, checks its version and wraps every
entry point so that tensors go in and a non-OK status becomes an exception with the library's message.

There is no other implementation behind these functions: when the library cannot be built or loaded, or when
no CUDA device is present, ``load()`` raises and nothing in the engine runs.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p

import torch

from . import build

ABI_VERSION = 11
F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dt} is neither float32 nor bfloat16")


def _ptr(t):
    """The address as a plain integer (ctypes converts it by the entry point's declared argument types)."""
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream's handle. The wrappers run hundreds of times a step, so this goes through torch's raw getter
    (a fraction of a microsecond) where the build has it, instead of building a Stream object (several microseconds)."""
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    return _raw_stream(torch.cuda.current_device())


def _need(t: torch.Tensor, name: str, dtype=None):
    if not t.is_cuda:
        raise KernelError(f"{name} is not on a CUDA device")
    if not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}; expected {dtype}")


_SIGNATURES = {
    "roost_status_snapshot": [c_void_p, c_int, c_void_p],
    "roost_embedding": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "roost_rms_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p],
    "roost_add_rms_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p],
    "roost_silu_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "roost_gemm_tcgen05_swiglu": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_void_p],
    "roost_qk_norm_rope_cache": [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int64, c_int, c_int, c_int,
                                 c_void_p],
    "roost_rope_table": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "roost_paged_attention_generic": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                      c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
    "roost_attention_mma_supported": [c_int],
    "roost_attention_prefill_tile_rows": [c_int, c_int, c_int, c_int, ctypes.c_longlong, c_void_p, c_void_p, ctypes.c_longlong],
    "roost_attention_set_prefill_tc": [c_int],
    "roost_attention_prefill": [c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_int, c_int, c_int, c_int, c_int, c_int, ctypes.c_longlong, c_float, c_int, c_void_p],
    "roost_attention_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                               c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, ctypes.c_longlong, c_float, c_int,
                               c_void_p],
    "roost_attention_decode_cluster": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                       c_int, c_int, c_int, c_int, ctypes.c_longlong, c_float, c_int, c_void_p],
    "roost_attention_decode_cluster_supported": [c_int, c_int, ctypes.c_longlong, c_int, c_void_p, c_void_p],
    "roost_sample_penalise": [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_void_p],
    "roost_sample_count_tokens": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p],
    "roost_sample_prompt_bits": [c_void_p, c_void_p, c_int, c_int, c_void_p],
    "roost_sample_logprobs": [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p],
    "roost_gemm_simt": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_void_p],
    "roost_gemm_tcgen05_supported": [c_int, c_int, c_int, c_int64, c_int64],
    "roost_gemm_tcgen05": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_void_p],
    "roost_gemm_tcgen05_status": [],
    "roost_attention_status": [],
    "roost_attention_set_decode_tma": [c_int],
    "roost_gemm_stream_workspace_floats": [],
    "roost_gemm_stream_workspace_flags": [],
    "roost_gemm_stream_supported": [c_int, c_int, c_int, c_int64, c_int64],
    "roost_gemm_split_supported": [c_int, c_int, c_int, c_int64, c_int64],
    "roost_gemm_split_preferred": [c_int, c_int, c_int, c_int64, c_int64],
    "roost_gemm_split_swiglu_supported": [c_int, c_int, c_int, c_int64, c_int64],
    "roost_gemm_split_swiglu": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_void_p],
    "roost_gemm_split": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_void_p],
    "roost_gemm_stream": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p,
                          c_void_p],
    "roost_gemm_stream_swiglu_supported": [c_int, c_int, c_int, c_int64, c_int64],
    "roost_gemm_stream_swiglu": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p,
                                 c_void_p],
    "roost_argmax": [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p],
    "roost_argmax_split": [c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "roost_sample": [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                     c_void_p, c_void_p],
}


class KernelLibrary:
    def __init__(self, path):
        self.path = str(path)
        self._lib = ctypes.CDLL(self.path)
        self._lib.roost_abi_version.restype = c_int
        self._lib.roost_last_error.restype = c_char_p
        got = self._lib.roost_abi_version()
        if got != ABI_VERSION:
            raise KernelError(f"{self.path} has ABI version {got}; this package needs {ABI_VERSION}")
        for name, args in _SIGNATURES.items():
            fn = getattr(self._lib, name)
            fn.argtypes = args
            fn.restype = c_int
        self.decode_chunk = 512  # keys per work item of the split decode attention (see decode_chunk_for)
        self.decode_cluster = True  # split rows merged by thread-block clusters where they fit (see decode_cluster_for)
        self._decode_ctas = 0
        self.launches = 0  # kernels launched through this handle (a host-side count of entry-point calls that launch)
        self.library_launches = 0  # products handed to cuBLAS through torch beside them (counted where they are called)

    def _call(self, name: str, *args, launches: int = 1):
        status = getattr(self._lib, name)(*args)
        if status != 0:
            msg = self._lib.roost_last_error().decode(errors="replace")
            raise KernelError(f"{name}: {msg} (status {status})")
        self.launches += launches

    def decode_chunk_for(self, rows: int, kv_cap: int, kv_heads: int) -> int:
        """Keys per work item of the split decode attention for a step of ``rows`` rows whose requests hold at most
        ``kv_cap`` keys (the bound of the captured step, so that every replay of it agrees). The persistent decode
        kernel runs two CTAs an SM; when ``decode_chunk`` keys an item give more items than CTAs but at most twice as
        many, the second round would be half empty, and items of twice the keys run as one full round instead (batch 8
        at 4096 keys: 4.42 against 4.51 ms a step). A row's bits then depend on the step's size class, within rounding."""
        if not self._decode_ctas:
            self._decode_ctas = 2 * torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        items = rows * kv_heads * (-(-max(kv_cap, 1) // self.decode_chunk))
        return 2 * self.decode_chunk if self._decode_ctas < items <= 2 * self._decode_ctas else self.decode_chunk

    def decode_cluster_for(self, rows: int, kv_cap: int, chunk: int, k_pool: torch.Tensor, v_pool: torch.Tensor) -> int:
        """CTAs of a cluster that takes one (row, key/value head) of the split decode attention and merges the row's
        chunks itself, for a step of ``rows`` rows whose requests hold at most ``kv_cap`` keys in chunks of ``chunk``: the
        power of two that covers the chunks, when that is 2 to 8 and all the clusters run at once (two CTAs an SM);
        else 0: partial results go through memory and the merge kernel. Same bits either way."""
        if not self.decode_cluster:
            return 0
        if not self._decode_ctas:
            self._decode_ctas = 2 * torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        pages, nkv, page, d = k_pool.shape
        chunks = -(-max(kv_cap, 1) // chunk)
        size = 1
        while size < chunks:
            size *= 2
        if size < 2 or size > 8 or rows * nkv * size > self._decode_ctas:
            return 0
        return size if self._lib.roost_attention_decode_cluster_supported(d, page, pages, nkv, _ptr(k_pool), _ptr(v_pool)) else 0

    def decode_split_for(self, rows: int, kv_cap: int, k_pool: torch.Tensor, v_pool: torch.Tensor) -> tuple[int, int]:
        """(keys per work item, CTAs a cluster or 0) of the split decode attention for a step of ``rows`` rows whose
        requests hold at most ``kv_cap`` keys (the bounds of the captured step, so that every replay of it agrees). Where
        clusters serve, the smallest chunk of 128, 256, 512 or 1024 keys whose clusters all run at once: more CTAs pull
        on the memory and the merge costs no kernel (one row of 1,024 keys: 7.7 us in chunks of 128, 12.6 us in chunks of
        512). Else the chunk of ``decode_chunk_for`` through the merge kernel. A row's bits depend on the chunk, so on
        the step's size class, within rounding."""
        if self.decode_cluster and kv_cap > 0:
            for chunk in (128, 256, 512, 1024):
                cluster = self.decode_cluster_for(rows, kv_cap, chunk, k_pool, v_pool)
                if cluster:
                    return chunk, cluster
        return self.decode_chunk_for(rows, kv_cap, k_pool.shape[1]), 0

    # ------------------------------------------------------------------ ops
    def embedding(self, table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        _need(table, "table"); _need(ids, "ids", torch.int32)
        T, (V, H) = ids.numel(), table.shape
        out = torch.empty((T, H), dtype=table.dtype, device=table.device)
        self._call("roost_embedding", _ptr(table), _ptr(ids), _ptr(out), T, H, V, dtype_code(table.dtype), _stream())
        return out

    def rms_norm(self, x: torch.Tensor, w: torch.Tensor, eps: float, rows: torch.Tensor | None = None) -> torch.Tensor:
        _need(x, "x"); _need(w, "w")
        H = x.shape[-1]
        if w.numel() != H:
            raise KernelError(f"rms_norm: weight has {w.numel()} elements for rows of {H}")
        n = x.numel() // H if rows is None else rows.numel()
        out = torch.empty((n, H) if rows is not None else x.shape, dtype=x.dtype, device=x.device)
        self._call("roost_rms_norm", _ptr(x), _ptr(w), _ptr(out), _ptr(rows), n, H, eps, dtype_code(x.dtype),
                   dtype_code(w.dtype), _stream())
        return out

    def add_rms_norm(self, x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float,
                     rows: torch.Tensor | None = None) -> torch.Tensor:
        """residual += x (in place, unless ``rows`` gathers) and the norm of the sum."""
        _need(x, "x"); _need(residual, "residual", x.dtype); _need(w, "w")
        H = x.shape[-1]
        if residual.shape != x.shape or w.numel() != H:
            raise KernelError("add_rms_norm: x, residual and weight do not agree in shape")
        n = x.numel() // H if rows is None else rows.numel()
        out = torch.empty((n, H), dtype=x.dtype, device=x.device)
        self._call("roost_add_rms_norm", _ptr(x), _ptr(residual), _ptr(w), _ptr(out), _ptr(rows), n, H, eps,
                   dtype_code(x.dtype), dtype_code(w.dtype), _stream())
        return out

    def silu_mul(self, x: torch.Tensor, block: int = 0) -> torch.Tensor:
        """silu(gate) * up over rows [gate | up] (block 0) or rows of blocks of ``block`` gate then ``block`` up values."""
        _need(x, "x")
        T, two_i = x.shape
        out = torch.empty((T, two_i // 2), dtype=x.dtype, device=x.device)
        self._call("roost_silu_mul", _ptr(x), _ptr(out), T, two_i // 2, block, dtype_code(x.dtype), _stream())
        return out

    def gemm_tcgen05_swiglu(self, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """silu(a Wg^T) * (a Wu^T) in one kernel; w holds gate and up rows interleaved in blocks of 128."""
        _need(a, "a", torch.bfloat16); _need(w, "w", torch.bfloat16)
        M, K = a.shape
        N, K2 = w.shape
        if K != K2:
            raise KernelError(f"gemm_tcgen05_swiglu: a has {K} columns, w has {K2}")
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device)
        self._call("roost_gemm_tcgen05_swiglu", _ptr(a), _ptr(w), _ptr(out), M, N, K, a.stride(0), w.stride(0), out.stride(0), _stream())
        return out

    def rope_table(self, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
        """(cos, sin) of positions[t] * inv_freq[i] as float32 [T, half, 2]: a step computes it once for all its layers."""
        _need(positions, "positions", torch.int32); _need(inv_freq, "inv_freq", torch.float64)
        T, half = positions.numel(), inv_freq.numel()
        out = torch.empty((T, half, 2), dtype=torch.float32, device=positions.device)
        self._call("roost_rope_table", _ptr(positions), _ptr(inv_freq), T, half, _ptr(out), _stream())
        return out

    def qk_norm_rope_cache(self, qkv, q_heads, kv_heads, head_dim, *, q_w, k_w, eps, inv_freq, rotary_dim, positions,
                           k_pool=None, v_pool=None, slot_mapping=None, page_size=0, write_kv=True, cos_sin=None) -> torch.Tensor:
        """qkv: [T, (q_heads + 2 kv_heads) * head_dim] (or [T, q_heads * head_dim] with write_kv False). Returns
        q: [T, q_heads, head_dim], normed and rotated; k and v go into the pools. ``cos_sin``: the step's table from
        ``rope_table`` for these positions and this ``inv_freq`` (else the kernel computes the same values itself)."""
        _need(qkv, "qkv")
        T = qkv.shape[0]
        width = (q_heads + (2 * kv_heads if write_kv else 0)) * head_dim
        if qkv.shape[1] != width:
            raise KernelError(f"qk_norm_rope_cache: qkv rows have {qkv.shape[1]} elements; expected {width}")
        q = torch.empty((T, q_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
        wd = dtype_code(q_w.dtype) if q_w is not None else F32
        pages = 0
        if write_kv:
            _need(k_pool, "k_pool", qkv.dtype); _need(v_pool, "v_pool", qkv.dtype); _need(slot_mapping, "slot_mapping", torch.int32)
            pages = k_pool.shape[0]
            if tuple(k_pool.shape[1:]) != (kv_heads, page_size, head_dim) or k_pool.shape != v_pool.shape:
                raise KernelError(f"qk_norm_rope_cache: pool shape {tuple(k_pool.shape)} is not [pages, {kv_heads}, {page_size}, {head_dim}]")
        if rotary_dim:
            _need(inv_freq, "inv_freq", torch.float64); _need(positions, "positions", torch.int32)
            if inv_freq.numel() != rotary_dim // 2:
                raise KernelError("qk_norm_rope_cache: inv_freq must have rotary_dim / 2 entries")
            if cos_sin is not None:
                _need(cos_sin, "cos_sin", torch.float32)
                if tuple(cos_sin.shape) != (T, rotary_dim // 2, 2):
                    raise KernelError(f"qk_norm_rope_cache: the table is {tuple(cos_sin.shape)}; expected {(T, rotary_dim // 2, 2)}")
        else:
            cos_sin = None
        self._call("roost_qk_norm_rope_cache", _ptr(qkv), qkv.stride(0), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(q_w),
                   _ptr(k_w), _ptr(inv_freq), _ptr(positions), _ptr(slot_mapping), _ptr(cos_sin), T, q_heads, kv_heads, head_dim,
                   rotary_dim, eps, page_size, pages, 1 if write_kv else 0, dtype_code(qkv.dtype), wd, _stream())
        return q

    def paged_attention_generic(self, q, k_pool, v_pool, positions, token_row, kv_indptr, kv_indices, scale: float,
                                window: int | None) -> torch.Tensor:
        _need(q, "q"); _need(k_pool, "k_pool", q.dtype); _need(v_pool, "v_pool", q.dtype)
        for n, t in (("positions", positions), ("token_row", token_row), ("kv_indptr", kv_indptr), ("kv_indices", kv_indices)):
            _need(t, n, torch.int32)
        T, nq, d = q.shape
        _, nkv, page, d2 = k_pool.shape
        if d2 != d:
            raise KernelError("paged_attention: head_dim of q and of the pool differ")
        out = torch.empty((T, nq * d), dtype=q.dtype, device=q.device)
        self._call("roost_paged_attention_generic", _ptr(q), _ptr(out), _ptr(k_pool), _ptr(v_pool), _ptr(positions),
                   _ptr(token_row), _ptr(kv_indptr), _ptr(kv_indices), T, nq, nkv, d, page, scale,
                   int(window) if window else 0, dtype_code(q.dtype), _stream())
        return out

    def attention_mma_supported(self, head_dim: int) -> bool:
        return bool(self._lib.roost_attention_mma_supported(int(head_dim)))

    def attention_prefill_tile_rows(self, q_heads: int, k_pool: torch.Tensor, v_pool: torch.Tensor, packed_rows: int = 0) -> int:
        """Packed rows of a prefill work item (64 or 128) for these pools [pages, kv_heads, page_size, head_dim] and a step
        that brings ``packed_rows`` packed rows in all to the prefill kernels."""
        pages, nkv, page, d = k_pool.shape
        return int(self._lib.roost_attention_prefill_tile_rows(d, int(q_heads), nkv, page, pages, _ptr(k_pool), _ptr(v_pool), int(packed_rows)))

    def attention_set_prefill_tc(self, on: bool) -> None:
        """Prompt portions run the tcgen05 attention kernel where the sizes allow (the default), or never."""
        self._lib.roost_attention_set_prefill_tc(1 if on else 0)

    def attention_mma(self, q, k_pool, v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, plan, scale: float,
                      window: int | None) -> torch.Tensor:
        """Tensor-core attention (bfloat16). ``plan``: an ``AttentionPlan`` whose work lists are on the device."""
        _need(q, "q", torch.bfloat16); _need(k_pool, "k_pool", torch.bfloat16); _need(v_pool, "v_pool", torch.bfloat16)
        T, nq, d = q.shape
        _, nkv, page, d2 = k_pool.shape
        if d2 != d:
            raise KernelError("attention_mma: head_dim of q and of the pool differ")
        out = torch.empty((T, nq * d), dtype=q.dtype, device=q.device)
        w = int(window) if window else 0
        if plan.prefill_items:
            self._call("roost_attention_prefill", _ptr(q), T, _ptr(out), _ptr(k_pool), _ptr(v_pool), _ptr(q_indptr), _ptr(kv_lens),
                       _ptr(kv_indptr), _ptr(kv_indices), _ptr(plan.prefill_work), plan.prefill_items, plan.prefill_tile_rows, nq, nkv, d, page,
                       k_pool.shape[0], scale, w, _stream())
        if plan.decode_items and plan.cluster_chunks:
            self._call("roost_attention_decode_cluster", _ptr(q), _ptr(out), _ptr(k_pool), _ptr(v_pool), _ptr(q_indptr), _ptr(kv_lens),
                       _ptr(kv_indptr), _ptr(kv_indices), _ptr(plan.decode_work), plan.decode_items, plan.cluster_chunks, nq, nkv, d, page,
                       k_pool.shape[0], scale, w, _stream())
        elif plan.decode_items:
            part_o = part_ml = None
            if plan.slots:
                part_o = torch.empty((plan.slots * nkv * 16 * d,), dtype=torch.float32, device=q.device)
                part_ml = torch.empty((plan.slots * nkv * 16 * 2,), dtype=torch.float32, device=q.device)
            self._call("roost_attention_decode", _ptr(q), _ptr(out), _ptr(k_pool), _ptr(v_pool), _ptr(q_indptr), _ptr(kv_lens),
                       _ptr(kv_indptr), _ptr(kv_indices), _ptr(plan.decode_work), plan.decode_items, _ptr(plan.merge_work),
                       plan.merge_items, plan.merge_rows, _ptr(part_o), _ptr(part_ml), nq, nkv, d, page, k_pool.shape[0], scale, w, _stream(),
                       launches=2 if plan.merge_items else 1)
        return out

    def gemm_simt(self, a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """a [M, K] times w [N, K] transposed, 32-bit FFMA accumulation."""
        _need(a, "a"); _need(w, "w", a.dtype)
        M, K = a.shape
        N, K2 = w.shape
        if K != K2:
            raise KernelError(f"gemm: a has {K} columns, w has {K2}")
        out_dtype = out_dtype or a.dtype
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        self._call("roost_gemm_simt", _ptr(a), _ptr(w), _ptr(out), M, N, K, a.stride(0), w.stride(0), out.stride(0),
                   dtype_code(a.dtype), dtype_code(out_dtype), _stream())
        return out

    def gemm_tcgen05_supported(self, m: int, n: int, k: int, lda: int, ldw: int) -> bool:
        return bool(self._lib.roost_gemm_tcgen05_supported(m, n, k, lda, ldw))

    def gemm_tcgen05(self, a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """a [M, K] times w [N, K] transposed on the tcgen05 tensor cores (TMA loads, accumulator in tensor memory)."""
        _need(a, "a", torch.bfloat16); _need(w, "w", torch.bfloat16)
        M, K = a.shape
        N, K2 = w.shape
        if K != K2:
            raise KernelError(f"gemm_tcgen05: a has {K} columns, w has {K2}")
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        self._call("roost_gemm_tcgen05", _ptr(a), _ptr(w), _ptr(out), M, N, K, a.stride(0), w.stride(0), out.stride(0),
                   dtype_code(out_dtype), _stream())
        return out

    def set_pdl(self, on: bool) -> None:
        """Programmatic dependent launch for the library's kernels."""
        self._lib.roost_set_pdl(1 if on else 0)
        self.pdl = bool(on)

    def gemm_stream_supported(self, m: int, n: int, k: int, ldx: int, ldw: int) -> bool:
        return bool(self._lib.roost_gemm_stream_supported(m, n, k, ldx, ldw))

    def _stream_workspace(self, device):
        ws = getattr(self, "_stream_ws", None)
        if ws is None or ws[0].device != device:
            # allocated once, outside any stream capture (the first decode step of a model runs eagerly)
            ws = self._stream_ws = (torch.zeros(self._lib.roost_gemm_stream_workspace_floats(), dtype=torch.float32, device=device),
                                    torch.zeros(self._lib.roost_gemm_stream_workspace_flags(), dtype=torch.int32, device=device))
        return ws

    def gemm_stream(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """x [M <= 64, K] times w [N, K] transposed: the weight-streaming tcgen05 product of decode steps."""
        _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16)
        M, K = x.shape
        N, K2 = w.shape
        if K != K2:
            raise KernelError(f"gemm_stream: x has {K} columns, w has {K2}")
        ws = self._stream_workspace(x.device)
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        self._call("roost_gemm_stream", _ptr(x), _ptr(w), _ptr(out), M, N, K, x.stride(0), w.stride(0), out.stride(0),
                   dtype_code(out_dtype), _ptr(ws[0]), _ptr(ws[1]), _stream())
        return out

    def gemm_split_supported(self, m: int, n: int, k: int, ldx: int, ldw: int) -> bool:
        return bool(self._lib.roost_gemm_split_supported(m, n, k, ldx, ldw))

    def gemm_split_preferred(self, m: int, n: int, k: int, ldx: int, ldw: int) -> bool:
        """Whether the k-split product was measured faster than the other products for this shape."""
        return bool(self._lib.roost_gemm_split_preferred(m, n, k, ldx, ldw))

    def gemm_split(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """x [M <= 64, K] times w [N, K] transposed for a weight of few 128-row tiles and a long K: K split over
        thread-block clusters, the partial sums added up through distributed shared memory."""
        _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16)
        M, K = x.shape
        N, K2 = w.shape
        if K != K2:
            raise KernelError(f"gemm_split: x has {K} columns, w has {K2}")
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        self._call("roost_gemm_split", _ptr(x), _ptr(w), _ptr(out), M, N, K, x.stride(0), w.stride(0), out.stride(0),
                   dtype_code(out_dtype), _stream())
        return out

    def gemm_split_swiglu_supported(self, m: int, n: int, k: int, ldx: int, ldw: int) -> bool:
        return bool(self._lib.roost_gemm_split_swiglu_supported(m, n, k, ldx, ldw))

    def gemm_split_swiglu(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """silu(x Wg^T) * (x Wu^T) for x [M <= 32, K] and w [2I, K] with gate and up rows interleaved in blocks of 128:
        the k-split product with the activation applied to the summed accumulators; returns [M, I]."""
        _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16)
        M, K = x.shape
        N, K2 = w.shape
        if K != K2:
            raise KernelError(f"gemm_split_swiglu: x has {K} columns, w has {K2}")
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((M, N // 2), dtype=out_dtype, device=x.device)
        self._call("roost_gemm_split_swiglu", _ptr(x), _ptr(w), _ptr(out), M, N, K, x.stride(0), w.stride(0), out.stride(0),
                   dtype_code(out_dtype), _stream())
        return out

    def gemm_stream_swiglu_supported(self, m: int, n: int, k: int, ldx: int, ldw: int) -> bool:
        return bool(self._lib.roost_gemm_stream_swiglu_supported(m, n, k, ldx, ldw))

    def gemm_stream_swiglu(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """silu(x Wg^T) * (x Wu^T) for x [M <= 32, K] and w [2I, K] with gate and up rows interleaved in blocks of 128:
        the weight-streaming product with the activation applied to its accumulators; returns [M, I]."""
        _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16)
        M, K = x.shape
        N, K2 = w.shape
        if K != K2:
            raise KernelError(f"gemm_stream_swiglu: x has {K} columns, w has {K2}")
        ws = self._stream_workspace(x.device)
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((M, N // 2), dtype=out_dtype, device=x.device)
        self._call("roost_gemm_stream_swiglu", _ptr(x), _ptr(w), _ptr(out), M, N, K, x.stride(0), w.stride(0), out.stride(0),
                   dtype_code(out_dtype), _ptr(ws[0]), _ptr(ws[1]), _stream())
        return out

    def attention_set_decode_tma(self, on: bool) -> None:
        """Decode rows stream keys and values through the copy engine where the sizes allow (the default), or never."""
        self._lib.roost_attention_set_decode_tma(1 if on else 0)

    def attention_status(self) -> int:
        """The code of a bounded wait the copy-engine decode kernel gave up since the last call (0: none); synchronises."""
        return int(self._lib.roost_attention_status())

    def status_snapshot(self, out: torch.Tensor) -> None:
        """Writes the kernels' error words into ``out`` (four int32: three codes, then 1) in stream order, without
        synchronising. ``out`` is on the device or in pinned host memory: an engine that copies a step's tokens to the
        host puts the words beside them and reads both after the one wait it makes anyway."""
        if out.dtype != torch.int32 or out.numel() < 4 or not out.is_contiguous():
            raise KernelError("status_snapshot: four contiguous int32 are needed")
        if not out.is_cuda and not out.is_pinned():
            raise KernelError("status_snapshot: a host destination must be pinned memory")
        self._call("roost_status_snapshot", _ptr(out), 0 if out.is_cuda else 1, _stream())

    def check_device_status(self) -> None:
        """Raises when a kernel gave up one of its bounded waits since the last call (its results are then not valid).
        Synchronises, clears the error words and lowers the flags a weight-streaming product that gave up may have left
        raised, so that the launches after the error start clean."""
        gemm, attn = self.gemm_tcgen05_status(), self.attention_status()
        if gemm or attn:
            ws = getattr(self, "_stream_ws", None)
            if ws is not None:
                ws[1].zero_()
            raise KernelError(f"a kernel gave up a bounded wait (tcgen05 product: code {gemm}, decode attention: code {attn}); "
                              "the step's results are not valid")

    def gemm_tcgen05_set_pairs(self, on: bool) -> None:
        """Tiles on pairs of CTAs (cta_group::2, the default) or on single CTAs."""
        self._lib.roost_gemm_tcgen05_set_pairs(1 if on else 0)

    def gemm_tcgen05_status(self) -> int:
        """The code of a bounded wait the tcgen05 product gave up since the last call (0: none); synchronises."""
        return int(self._lib.roost_gemm_tcgen05_status())

    def argmax(self, logits: torch.Tensor) -> torch.Tensor:
        _need(logits, "logits", torch.float32)
        R, V = logits.shape
        ids = torch.empty((R,), dtype=torch.int32, device=logits.device)
        splits = min(16, V // 8192)     # a block a span of 8192 logits or more, up to 16 blocks a row
        if splits > 1:
            ws = getattr(self, "_argmax_ws", None)
            if ws is None or ws[2].numel() < R or ws[2].device != logits.device:
                cap = max(64, R)
                ws = self._argmax_ws = (torch.empty(cap * 16, dtype=torch.float32, device=logits.device),
                                        torch.empty(cap * 16, dtype=torch.int32, device=logits.device),
                                        torch.zeros(cap, dtype=torch.int32, device=logits.device))
            self._call("roost_argmax_split", _ptr(logits), logits.stride(0), R, V, _ptr(ids), splits, _ptr(ws[0]), _ptr(ws[1]), _ptr(ws[2]),
                       _stream())
            return ids
        self._call("roost_argmax", _ptr(logits), logits.stride(0), R, V, _ptr(ids), _stream())
        return ids

    def sample(self, logits, temperature, top_k, top_p, min_p, seeds, offsets, workspace=None) -> torch.Tensor:
        _need(logits, "logits", torch.float32)
        R, V = logits.shape
        for n, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32), ("top_p", top_p, torch.float32),
                         ("min_p", min_p, torch.float32), ("seeds", seeds, torch.int64), ("offsets", offsets, torch.int64)):
            _need(t, n, dt)
            if t.numel() != R:
                raise KernelError(f"sample: {n} has {t.numel()} entries for {R} rows")
        if workspace is None:
            workspace = torch.empty((R, V), dtype=torch.float32, device=logits.device)
        ids = torch.empty((R,), dtype=torch.int32, device=logits.device)
        self._call("roost_sample", _ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(top_k), _ptr(top_p),
                   _ptr(min_p), _ptr(seeds), _ptr(offsets), _ptr(workspace), _ptr(ids), _stream())
        return ids

    def sample_penalise(self, logits, counts, prompt_bits, row_slot, repetition, presence, frequency, mask_bits=None) -> torch.Tensor:
        """The rows of ``logits`` with the reference's repetition, frequency and presence penalties applied: counts
        [slots, vocab] int32 (the requests' output tokens so far), prompt_bits [slots, (vocab + 31) // 32] int32 (the
        prompts' tokens), row_slot [rows] int32 (-1: the row is copied as it is), the penalties float32 [rows]; then
        -inf where a token's bit in mask_bits (shaped as prompt_bits; None: every token stays) is 0."""
        _need(logits, "logits", torch.float32); _need(counts, "counts", torch.int32); _need(prompt_bits, "prompt_bits", torch.int32)
        R, V = logits.shape
        if counts.shape[1] != V or prompt_bits.shape != (counts.shape[0], (V + 31) // 32):
            raise KernelError(f"sample_penalise: counts {tuple(counts.shape)} and prompt_bits {tuple(prompt_bits.shape)} do not fit a vocabulary of {V}")
        for n, t, dt in (("row_slot", row_slot, torch.int32), ("repetition", repetition, torch.float32), ("presence", presence, torch.float32),
                         ("frequency", frequency, torch.float32)):
            _need(t, n, dt)
            if t.numel() != R:
                raise KernelError(f"sample_penalise: {n} has {t.numel()} entries for {R} rows")
        out = torch.empty((R, V), dtype=torch.float32, device=logits.device)
        if mask_bits is not None:
            _need(mask_bits, "mask_bits", torch.int32)
            if mask_bits.shape != prompt_bits.shape:
                raise KernelError("sample_penalise: mask_bits must be shaped as prompt_bits")
        self._call("roost_sample_penalise", _ptr(logits), logits.stride(0), R, V, _ptr(out), _ptr(counts), _ptr(prompt_bits), _ptr(mask_bits),
                   _ptr(row_slot), _ptr(repetition), _ptr(presence), _ptr(frequency), _stream())
        return out

    def sample_count_tokens(self, counts, row_slot, ids) -> None:
        """counts[row_slot[r], ids[r]] += 1 for the rows with a slot and a token."""
        _need(counts, "counts", torch.int32); _need(row_slot, "row_slot", torch.int32); _need(ids, "ids", torch.int32)
        if row_slot.numel() != ids.numel():
            raise KernelError("sample_count_tokens: one slot a token id is needed")
        self._call("roost_sample_count_tokens", _ptr(counts), counts.shape[1], _ptr(row_slot), _ptr(ids), ids.numel(), _stream())

    def sample_prompt_bits(self, bits_of_slot, ids) -> None:
        """Sets the bits of the token ids ``ids`` in one slot's words (int32 [(vocab + 31) // 32], a view into the table)."""
        _need(bits_of_slot, "bits", torch.int32); _need(ids, "ids", torch.int32)
        self._call("roost_sample_prompt_bits", _ptr(bits_of_slot), _ptr(ids), ids.numel(), bits_of_slot.numel() * 32, _stream())

    def sample_logprobs(self, logits, ids, top: int = 0):
        """(log-softmax of the raw logits at ids [rows] float32, the ``top`` highest raw logits' ids [rows, top] int32 and
        their log-softmax [rows, top] float32), all on the device."""
        _need(logits, "logits", torch.float32); _need(ids, "ids", torch.int32)
        R, V = logits.shape
        if ids.numel() != R or not 0 <= top <= V:
            raise KernelError(f"sample_logprobs: {ids.numel()} ids for {R} rows, or top {top} outside [0, {V}]")
        lp = torch.empty((R,), dtype=torch.float32, device=logits.device)
        top_ids = torch.empty((R, top), dtype=torch.int32, device=logits.device)
        top_vals = torch.empty((R, top), dtype=torch.float32, device=logits.device)
        self._call("roost_sample_logprobs", _ptr(logits), logits.stride(0), R, V, _ptr(ids), _ptr(lp), top, _ptr(top_ids) if top else None,
                   _ptr(top_vals) if top else None, _stream())
        return lp, top_ids, top_vals


_LIB: KernelLibrary | None = None


def load() -> KernelLibrary:
    """The process-wide library handle. Raises when no CUDA device is present or the library cannot be built."""
    global _LIB
    if _LIB is None:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is visible: roost_b200 runs on an sm_100a GPU only and has no CPU path")
        major, minor = torch.cuda.get_device_capability()
        if major != 10:
            raise KernelError(f"the GPU has compute capability {major}.{minor}; the kernel library is built for sm_100a only")
        _LIB = KernelLibrary(build.library_path())
        import os
        # The bfloat16 products that go to cuBLAS through torch accumulate in 32-bit, as the reference asks of its library
        # (CUBLAS_COMPUTE_32F, kernels/src/gemm.cu:247-249). torch's default also lets a split-k product add its partial
        # sums up in bfloat16; that is switched off here, so that every sum of the bfloat16 path is a 32-bit sum.
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        # programmatic dependent launch is on unless ROOST_PDL=0: the library's kernels overlap their preambles, and the
        # weight-streaming product its first loads of weights, with the tail of the kernel before them
        _LIB.set_pdl(os.environ.get("ROOST_PDL", "1") != "0")
        _LIB.decode_cluster = os.environ.get("ROOST_DECODE_CLUSTER", "1") != "0"
    return _LIB
