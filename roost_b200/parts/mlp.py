"""The gated feed-forward: down(act(x Wg^T) * (x Wu^T)), gate and up as one product over the row-wise
concatenation [gate; up] made at load (src/Starlings.Roost.Models.Tiny/RoostTiny.cs:35-36,51-53;
silu(g) = g / (1 + exp(-g)), src/Starlings.Roost.Ops/CpuOps.cs:355-368)."""
from __future__ import annotations

from ..config.spec import GatedMlpSpec
from .base import FeedForward, ParamDecl, Runtime, register_feed_forward
from .linear import Linear


class GatedMlp(FeedForward):
    def __init__(self, spec: GatedMlpSpec, runtime: Runtime):
        if spec.hidden <= 0 or spec.intermediate <= 0:
            raise ValueError("gated_mlp: hidden and intermediate must be positive")
        if spec.activation != "silu":
            raise ValueError(f"gated_mlp: activation '{spec.activation}' has no kernel (built: silu)")
        self.spec = spec
        self.rt = runtime
        self.gate_up = Linear(runtime, 2 * spec.intermediate, spec.hidden)
        self.down = Linear(runtime, spec.hidden, spec.intermediate)
        # In bfloat16 with an intermediate size that is a multiple of 128 the gate and up rows are stored interleaved in
        # blocks of 128, the layout in which the tensor-core product applies SiLU(gate) * up to its accumulator, so that
        # for many rows of x the [T, 2I] product never goes to memory; few rows keep the library product and the
        # SiLU kernel, which reads the same layout.
        k = runtime.kernels
        self.interleave = 128 if (not runtime.full_precision and spec.intermediate % 128 == 0 and spec.hidden % 8 == 0
                                  and hasattr(k, "gemm_tcgen05_swiglu")) else 0
        self.fused_min_rows = 256   # below this the 128-row tiles are mostly empty and the library product is faster
        # ... and so it is while the product is small: measured on a B200, the library product followed by the SiLU kernel
        # wins at rows x intermediate x hidden below about 2.5e10 (hidden 1024, intermediate 3072: 12.9 against 19.4 us at
        # 512 rows, 32.5 against 39.5 at 2,048; hidden 4096, intermediate 12288: 55 against 62 us at 256 rows, even at 512)
        # and the fused product above it (281 against 303 us at 2,048 rows of the latter; 116 against 130 us at 256 rows
        # of hidden 5120, intermediate 25600).
        self.fused_min_work = 2.5e10
        # few rows (decode steps): the weight-streaming product can apply the activation too, which saves the SiLU kernel
        # and its round trip through memory. Measured on a B200 at the 8B layer sizes the library product followed by
        # the SiLU kernel is still 2 us a layer faster, so only the "stream" policy takes this path.
        self.fused_max_stream_rows = 16
        self.fused_stream_policies = ("stream",)
        # The same with the product whose k is split over thread-block clusters: at most 8 rows, where it was measured no
        # slower than the library product followed by the SiLU kernel at the 8B sizes (38.1 against 39.6 us alone; in
        # the step batch 1 at 1,024 keys 282 -> 293 tokens/s, batch 8 at 4,096 keys unchanged).
        self.fused_max_split_rows = 8
        self.fused_split_policies = ("split", "auto")

    @classmethod
    def parameters(cls, spec: GatedMlpSpec):
        I, H = spec.intermediate, spec.hidden
        return {"gate_up": ParamDecl(shape=(2 * I, H), row_splits=(I, I)), "down": ParamDecl(shape=(H, I))}

    def load(self, params):
        w = params["gate_up"]
        if self.interleave:
            I, H, b = self.spec.intermediate, self.spec.hidden, self.interleave
            w = w.reshape(2, I // b, b, H).permute(1, 0, 2, 3).reshape(2 * I, H)   # [gate; up] -> blocks of (gate, up)
        self.gate_up.load(w)
        self.down.load(params["down"])

    def __call__(self, x, batch=None):
        k = self.rt.kernels
        if (self.interleave and x.shape[0] >= self.fused_min_rows and x.is_contiguous()
                and float(x.shape[0]) * self.spec.intermediate * self.spec.hidden >= self.fused_min_work):
            return self.down(k.gemm_tcgen05_swiglu(x, self.gate_up.weight))
        if (self.interleave and x.shape[0] <= self.fused_max_split_rows and x.is_contiguous()
                and self.rt.small_gemm in self.fused_split_policies and hasattr(k, "gemm_split_swiglu")):
            w = self.gate_up.weight
            if k.gemm_split_swiglu_supported(x.shape[0], w.shape[0], w.shape[1], x.stride(0), w.stride(0)):
                return self.down(k.gemm_split_swiglu(x, w))    # decode steps: k split over clusters, activation on the sums
        if (self.interleave and x.shape[0] <= self.fused_max_stream_rows and x.is_contiguous()
                and self.rt.small_gemm in self.fused_stream_policies):
            w = self.gate_up.weight
            if k.gemm_stream_swiglu_supported(x.shape[0], w.shape[0], w.shape[1], x.stride(0), w.stride(0)):
                return self.down(k.gemm_stream_swiglu(x, w))   # decode steps: weights streamed once, activation in the epilogue
        return self.down(k.silu_mul(self.gate_up(x), self.interleave))


register_feed_forward("gated_mlp", GatedMlp)
