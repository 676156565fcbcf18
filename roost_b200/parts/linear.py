"""y = x W^T for a weight stored [out, in], no bias (src/Starlings.Roost.Ops/CpuOps.cs:395-437).

float32 runs the library's FFMA product (true 32-bit, the same bits for a row whatever the batch). bfloat16
with 32-bit accumulation goes to cuBLAS through torch, the place where the reference's engine also calls a
library (kernels/src/gemm.cu:235), except where a kernel of this library is faster. ``Runtime.small_gemm`` decides for
products of at most 64 rows (decode steps): "auto" takes this library's TMA/tcgen05 kernels where they were measured
faster than cuBLAS on a B200 (the product with k split over thread-block clusters for weights of few tiles and a long k:
output and down projections of at most 8 rows; the weight-streaming product for at most 16 rows and a reduction length
of 8192 or more, or the vocabulary-sized head) and leaves the rest to cuBLAS; "stream" and "split" force those kernels
wherever they serve, "library" forces cuBLAS.
"""
from __future__ import annotations

import torch

from .base import Runtime

_MM_OUT_DTYPE = None  # does torch.mm take out_dtype on this build? decided at first use


class Linear:
    def __init__(self, runtime: Runtime, out_features: int, in_features: int):
        self.rt = runtime
        self.out_features = out_features
        self.in_features = in_features
        self.weight: torch.Tensor | None = None

    def load(self, weight: torch.Tensor) -> None:
        if tuple(weight.shape) != (self.out_features, self.in_features):
            raise ValueError(f"linear: weight is {tuple(weight.shape)}; expected {(self.out_features, self.in_features)}")
        self.weight = weight.to(self.rt.dtype).contiguous()

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        global _MM_OUT_DTYPE
        k = self.rt.kernels
        out_dtype = out_dtype or self.rt.dtype
        if self.rt.full_precision:
            return k.gemm_simt(x, self.weight, torch.float32)
        M = x.shape[0]
        if M <= 64 and x.is_contiguous():
            policy = self.rt.small_gemm
            if policy in ("auto", "split") and getattr(k, "gemm_split_supported", None):
                choose = k.gemm_split_supported if policy == "split" else k.gemm_split_preferred
                if choose(M, self.out_features, self.in_features, x.stride(0), self.weight.stride(0)):
                    return k.gemm_split(x, self.weight, out_dtype)    # k split over thread-block clusters, tcgen05 products
            if policy == "stream" or (policy == "auto" and M <= 16 and (self.in_features >= 8192 or self.out_features >= 65536)):
                if k.gemm_stream_supported(M, self.out_features, self.in_features, x.stride(0), self.weight.stride(0)):
                    return k.gemm_stream(x, self.weight, out_dtype)   # weights streamed once by TMA, tcgen05 products
        if out_dtype == torch.bfloat16:
            k.library_launches += 1
            return torch.matmul(x, self.weight.t())
        if _MM_OUT_DTYPE is None:
            try:
                torch.mm(x[:1], self.weight[:8].t(), out_dtype=torch.float32)
                _MM_OUT_DTYPE = True
            except (TypeError, RuntimeError):
                _MM_OUT_DTYPE = False
        if _MM_OUT_DTYPE:
            k.library_launches += 1
            return torch.mm(x, self.weight.t(), out_dtype=torch.float32)
        return k.gemm_simt(x, self.weight, torch.float32)
