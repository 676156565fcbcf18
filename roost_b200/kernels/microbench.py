"""Times single kernels of the library on synthetic inputs, with CUDA events on the launching stream.

    python -m roost_b200.kernels.microbench attention-decode --batch 64 --context 4096
    python -m roost_b200.kernels.microbench attention-prefill --tokens 8192
    python -m roost_b200.kernels.microbench gemm-small --rows 8
    python -m roost_b200.kernels.microbench gemm-large --rows 2048
    python -m roost_b200.kernels.microbench sample --vocab 151936 --sample-rows 1,8,64

Each case prints one line per measurement: the time of one call, the achieved bandwidth or arithmetic rate, and what
the same bytes or operations would take at the device's measured peaks when a peak is given. The inputs are larger
than L2 (or rotate through several copies) so that DRAM figures mean something. It is the program the kernel profiles
under ``profiles/`` were taken with (``--iters 2 --warmup 1`` under a profiler).
"""
from __future__ import annotations

import argparse
import sys


def _time(fn, warmup: int, iters: int) -> float:
    """Microseconds of one call."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters * 1e3


def _graph_time(fns: list, warmup: int, iters: int) -> float:
    """Microseconds of one call when the calls of ``fns`` are replayed back to back from one CUDA graph."""
    import torch
    for f in fns:
        f()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for f in fns:
            f()
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns:
            f()
    return _time(g.replay, warmup, iters) / len(fns)


def attention_decode(k, a) -> None:
    import torch

    from ..parts.attention_work import plan_attention
    nq, nkv, d, page = a.q_heads, a.kv_heads, a.head_dim, a.page_size
    pages_per = -(-a.context // page)
    npages = pages_per * a.batch
    pool = torch.randn(2, npages, nkv, page, d, device="cuda", dtype=torch.bfloat16)   # keys then values, as the cache holds them
    q = torch.randn(a.batch, nq, d, device="cuda", dtype=torch.bfloat16)
    chunk, cluster = k.decode_split_for(a.batch, a.context, pool[0], pool[1])
    if a.chunk or a.no_cluster:
        chunk = a.chunk or k.decode_chunk_for(a.batch, a.context, nkv)
        cluster = 0 if a.no_cluster else k.decode_cluster_for(a.batch, a.context, chunk, pool[0], pool[1])
    plan = plan_attention([a.context - 1] * a.batch, [1] * a.batch, nq // nkv, None, chunk, "cuda", 64, cluster)
    q_indptr = torch.arange(a.batch + 1, dtype=torch.int32, device="cuda")
    kv_lens = torch.full((a.batch,), a.context, dtype=torch.int32, device="cuda")
    kv_indptr = torch.arange(a.batch + 1, dtype=torch.int32, device="cuda") * pages_per
    gen = torch.Generator(device="cuda").manual_seed(0)
    kv_indices = (torch.arange(npages, device="cuda") if a.sequential_pages else torch.randperm(npages, device="cuda", generator=gen)).to(torch.int32)
    k.attention_set_decode_tma(not a.cp_async)
    call = lambda: k.attention_mma(q, pool[0], pool[1], q_indptr, kv_lens, kv_indptr, kv_indices, plan, d ** -0.5, None)
    us = _time(call, a.warmup, a.iters)
    nbytes = a.batch * a.context * nkv * d * 2 * 2
    form = f"clusters of {cluster}" if cluster else "decode and merge kernels"
    print(f"attention-decode batch={a.batch} context={a.context} chunk={chunk} items={plan.decode_items} "
          f"{'cp.async' if a.cp_async else 'tma'}: {us:.1f} us, {nbytes / us / 1e6:.2f} TB/s of keys and values "
          f"({form}, eager launches), status {k.attention_status()}", flush=True)
    # replayed from a graph, calls on pools of their own (larger than L2 together where one is over 32 MB): no host time
    pools = [pool] + [torch.randn_like(pool) for _ in range(3)]
    calls = [(lambda p=p: k.attention_mma(q, p[0], p[1], q_indptr, kv_lens, kv_indptr, kv_indices, plan, d ** -0.5, None)) for p in pools]
    us = _graph_time(calls, a.warmup, a.iters)
    print(f"  in a graph of four calls over four pools: {us:.1f} us a call, {nbytes / us / 1e6:.2f} TB/s", flush=True)


def attention_prefill(k, a) -> None:
    import torch

    from ..parts.attention_work import plan_attention
    nq, nkv, d, page = a.q_heads, a.kv_heads, a.head_dim, a.page_size
    T = a.tokens
    pages_per = -(-T // page)
    npages = pages_per * a.batch
    pool = torch.randn(2, npages, nkv, page, d, device="cuda", dtype=torch.bfloat16)
    q = torch.randn(T * a.batch, nq, d, device="cuda", dtype=torch.bfloat16)
    group = nq // nkv
    k.attention_set_prefill_tc(not a.mma_sync)
    rows = a.tile_rows or k.attention_prefill_tile_rows(nq, pool[0], pool[1], T * a.batch * group)
    plan = plan_attention([0] * a.batch, [T] * a.batch, group, None, k.decode_chunk, "cuda", rows)
    q_indptr = torch.arange(a.batch + 1, dtype=torch.int32, device="cuda") * T
    kv_lens = torch.full((a.batch,), T, dtype=torch.int32, device="cuda")
    kv_indptr = torch.arange(a.batch + 1, dtype=torch.int32, device="cuda") * pages_per
    kv_indices = torch.randperm(npages, device="cuda").to(torch.int32)
    # replayed from a graph, several calls back to back: the host's part of a call (three tensor maps, the launch) is
    # then outside the measurement, as it is in a captured step
    call = lambda: k.attention_mma(q, pool[0], pool[1], q_indptr, kv_lens, kv_indptr, kv_indices, plan, d ** -0.5, None)
    us = _graph_time([call] * 4, a.warmup, a.iters)
    flops = 4 * T * T / 2 * nq * d * a.batch
    print(f"attention-prefill tokens={T} batch={a.batch} heads={nq}/{nkv} head_dim={d} tile_rows={rows} {'mma.sync' if a.mma_sync else 'tcgen05'}: {us:.1f} us, "
          f"{flops / us / 1e6:.0f} TFLOP/s (causal half counted)", flush=True)


def gemm_small(k, a) -> None:
    import torch
    shapes = [(a.n, a.k)] if a.n and a.k else [(6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288)]
    for n, kk in shapes:
        copies = max(4, int(600e6 // (n * kk * 2)))     # rotate through more than L2 holds
        ws = [torch.randn(n, kk, device="cuda", dtype=torch.bfloat16) for _ in range(copies)]
        x = torch.randn(a.rows, kk, device="cuda", dtype=torch.bfloat16)
        t_stream = _graph_time([(lambda w=w: k.gemm_stream(x, w)) for w in ws], a.warmup, a.iters)
        t_lib = _graph_time([(lambda w=w: torch.matmul(x, w.t())) for w in ws], a.warmup, a.iters)
        split = ""
        if k.gemm_split_supported(a.rows, n, kk, kk, kk):
            t_split = _graph_time([(lambda w=w: k.gemm_split(x, w)) for w in ws], a.warmup, a.iters)
            split = f"k split over clusters {t_split:.1f} us ({n * kk * 2 / t_split / 1e6:.2f} TB/s), "
        if n % 256 == 0 and k.gemm_split_swiglu_supported(a.rows, n, kk, kk, kk):
            t_sw = _graph_time([(lambda w=w: k.gemm_split_swiglu(x, w)) for w in ws], a.warmup, a.iters)
            t_two = _graph_time([(lambda w=w: k.silu_mul(torch.matmul(x, w.t()), 128)) for w in ws], a.warmup, a.iters)
            split += f"k split with SiLU x up {t_sw:.1f} us (cuBLAS and the SiLU kernel {t_two:.1f} us), "
        print(f"gemm-small rows={a.rows} n={n} k={kk}: stream {t_stream:.1f} us ({n * kk * 2 / t_stream / 1e6:.2f} TB/s of weights), {split}"
              f"cuBLAS {t_lib:.1f} us, in one graph back to back; status {k.gemm_tcgen05_status()}", flush=True)


def gemm_large(k, a) -> None:
    import torch
    shapes = [(a.n, a.k)] if a.n and a.k else [(6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288)]
    for n, kk in shapes:
        w = torch.randn(n, kk, device="cuda", dtype=torch.bfloat16)
        x = torch.randn(a.rows, kk, device="cuda", dtype=torch.bfloat16)
        flops = 2.0 * a.rows * n * kk
        for pairs in (True, False):
            k.gemm_tcgen05_set_pairs(pairs)
            us = _time(lambda: k.gemm_tcgen05(x, w), a.warmup, a.iters)
            print(f"gemm-large rows={a.rows} n={n} k={kk} tcgen05 {'CTA pairs' if pairs else 'single CTAs'}: {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s",
                  flush=True)
        k.gemm_tcgen05_set_pairs(True)
        us = _time(lambda: torch.matmul(x, w.t()), a.warmup, a.iters)
        print(f"gemm-large rows={a.rows} n={n} k={kk} cuBLAS: {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s; status {k.gemm_tcgen05_status()}", flush=True)


def sample(k, a) -> None:
    """The argmax and the sampling kernel over rows of a vocabulary's logits, at the batch sizes of the benchmark."""
    import torch
    V = a.vocab
    for rows in [int(x) for x in a.sample_rows.split(",")]:
        copies = max(2, int(300e6 // (rows * V * 4)))       # rotate through more than L2 holds
        logits = [torch.randn(rows, V, device="cuda") * 3 for _ in range(copies)]
        ws = torch.empty(rows, V, device="cuda")
        t = torch.full((rows,), a.temperature, device="cuda")
        tk = torch.full((rows,), a.top_k, dtype=torch.int32, device="cuda")
        tp = torch.full((rows,), a.top_p, device="cuda")
        mp = torch.zeros(rows, device="cuda")
        seeds = torch.arange(rows, dtype=torch.int64, device="cuda") + 99
        offs = torch.zeros(rows, dtype=torch.int64, device="cuda")
        turn = [0]

        def next_logits():
            turn[0] = (turn[0] + 1) % copies
            return logits[turn[0]]

        us_arg = _time(lambda: k.argmax(next_logits()), a.warmup, a.iters)
        us_smp = _time(lambda: k.sample(next_logits(), t, tk, tp, mp, seeds, offs, ws), a.warmup, a.iters)
        nbytes = rows * V * 4
        print(f"sample rows={rows} vocab={V} temperature={a.temperature} top_k={a.top_k} top_p={a.top_p}: argmax {us_arg:.1f} us "
              f"({nbytes / us_arg / 1e6:.2f} TB/s), sampler {us_smp:.1f} us ({nbytes / us_smp / 1e6:.3f} TB/s of one pass over the logits)", flush=True)


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m roost_b200.kernels.microbench", description=__doc__.split("\n")[0])
    p.add_argument("case", choices=["attention-decode", "attention-prefill", "gemm-small", "gemm-large", "sample"])
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=4096)
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--rows", type=int, default=8)
    p.add_argument("--n", type=int, default=0)
    p.add_argument("--k", type=int, default=0)
    p.add_argument("--q-heads", type=int, default=32)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--chunk", type=int, default=0, help="keys per decode work item (default: the library's)")
    p.add_argument("--no-cluster", action="store_true", help="split rows through partial results in memory and the merge kernel")
    p.add_argument("--tile-rows", type=int, default=0, help="packed rows per prefill work item: 64, 128 or 256 (default: the library's choice)")
    p.add_argument("--cp-async", action="store_true", help="decode attention through the cp.async kernel instead of TMA")
    p.add_argument("--mma-sync", action="store_true", help="prefill attention through the mma.sync kernel instead of tcgen05")
    p.add_argument("--sequential-pages", action="store_true")
    p.add_argument("--vocab", type=int, default=151936)
    p.add_argument("--sample-rows", default="1,8,64")
    p.add_argument("--temperature", type=float, default=0.8)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--top-p", type=float, default=0.9)
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    a = p.parse_args(argv)
    from . import library
    k = library.load()
    {"attention-decode": attention_decode, "attention-prefill": attention_prefill, "gemm-small": gemm_small, "gemm-large": gemm_large, "sample": sample}[a.case](k, a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
