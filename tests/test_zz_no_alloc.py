"""roost_attention_decode_static, the decode attention that takes no workspace, called through its exported C symbol.

The entry point is for hosts that cannot allocate device memory while they run: one that gave the whole GPU to its
own arena when it started, one whose step loop may never synchronise the device (cudaMalloc and cudaFree do), one that
is not allowed to grow its process's footprint. It keeps the partial results of split rows in a fixed 16 MiB array
inside the library. This test checks its output against roost_attention_decode, which takes caller-provided buffers,
on two calls in a row with different inputs (the array keeps the first call's contents when the second begins), that
the device's free memory is the same after each call as before it, that a work list naming more partial slots than
the caller declared is skipped and reported instead of written past the array, and that a request beyond the array's
size is refused. The file is named so that pytest collects it last.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _p(t):
    return None if t is None else c_void_p(t.data_ptr())


def test_decode_attention_without_a_workspace_matches_the_one_with(kernels):
    from roost_b200.parts.attention_work import plan_attention
    from tests.test_kernels_gpu import build_paged, close, paged_reference

    lib = ctypes.CDLL(kernels.path)
    fn = lib.roost_attention_decode_static
    fn.restype = c_int
    fn.argtypes = [c_void_p] * 9 + [c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]
    lib.roost_attention_decode_static_capacity_floats.restype = c_int
    lib.roost_last_error.restype = ctypes.c_char_p
    capacity = lib.roost_attention_decode_static_capacity_floats()
    assert capacity * 4 == 16 * 1024 * 1024

    dtype = torch.bfloat16
    nq, nkv, d, page = 8, 2, 128, 16
    scale = 1 / math.sqrt(d)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    free_around_calls = []
    for call, (lens, seed) in enumerate((([900, 300, 1200, 40], 31), ([517, 2049, 64], 32))):
        g = torch.Generator().manual_seed(seed)
        news = [1] * len(lens)
        keys = [torch.randn(n, nkv, d, generator=g).to(dtype).double() for n in lens]
        values = [torch.randn(n, nkv, d, generator=g).to(dtype).double() for n in lens]
        q = (torch.randn(len(lens), nq, d, generator=g) * 1.5).to(dtype).cuda()
        kp, vp, indptr, indices = build_paged(keys, values, page, dtype, num_pages=sum(-(-n // page) for n in lens) + 3, seed=seed)
        starts = [n - 1 for n in lens]
        plan = plan_attention(starts, news, nq // nkv, None, kernels.decode_chunk, "cuda", 64)
        assert plan.merge_items > 0 and plan.slots > 1
        q_indptr = torch.arange(len(lens) + 1, dtype=torch.int32).cuda()
        kv_lens = torch.tensor(lens, dtype=torch.int32).cuda()
        kernels.attention_set_decode_tma(False)   # the static entry point runs the cp.async kernel: compare like with like
        try:
            want = kernels.attention_mma(q, kp, vp, q_indptr, kv_lens, indptr, indices, plan, scale, None)
        finally:
            kernels.attention_set_decode_tma(True)
        got = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        free_around_calls.append(torch.cuda.mem_get_info()[0])
        rc = fn(_p(q), _p(got), _p(kp), _p(vp), _p(q_indptr), _p(kv_lens), _p(indptr), _p(indices), _p(plan.decode_work), plan.decode_items,
                _p(plan.merge_work), plan.merge_items, plan.slots, nq, nkv, d, page, scale, 0, stream)
        assert rc == 0, lib.roost_last_error().decode()
        torch.cuda.synchronize()
        # what the entry point is for: the device's free memory is the same after the call as before it (the test's own
        # tensors were all made before the first reading, and torch makes none inside the call)
        free_around_calls.append(torch.cuda.mem_get_info()[0])
        assert free_around_calls[-1] == free_around_calls[-2], "the call changed the device's free memory"
        close(got, want.double(), dtype, f"call {call}: static against workspace")
        assert torch.equal(got, want), "the same kernels on the same inputs give the same bits"
        positions = [n - 1 for n in lens]
        close(got, paged_reference(q.double().cpu(), keys, values, positions, list(range(len(lens))), scale, None), dtype,
              f"call {call}: static against the plain attention", scale=2)

    assert kernels.attention_status() == 0
    # a work list that names slots beyond `slots`: the items are skipped (their rows stay as they were) and the status
    # says so; nothing is written past the array
    got = torch.full_like(want, 7.0)
    rc = fn(_p(q), _p(got), _p(kp), _p(vp), _p(q_indptr), _p(kv_lens), _p(indptr), _p(indices), _p(plan.decode_work), plan.decode_items,
            _p(plan.merge_work), plan.merge_items, plan.slots - 1, nq, nkv, d, page, scale, 0, stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert kernels.attention_status() == 9 and kernels.attention_status() == 0
    assert bool((got.float() == 7.0).all(dim=1).any()), "the row whose last slot lies beyond the limit was merged all the same"

    # beyond the fixed array: refused with a clear error, nothing launched
    too_many = capacity // (nkv * 16 * d) + 1
    rc = fn(_p(q), _p(got), _p(kp), _p(vp), _p(q_indptr), _p(kv_lens), _p(indptr), _p(indices), _p(plan.decode_work), plan.decode_items,
            _p(plan.merge_work), plan.merge_items, too_many, nq, nkv, d, page, scale, 0, stream)
    assert rc == 2 and b"fixed array holds" in lib.roost_last_error()
