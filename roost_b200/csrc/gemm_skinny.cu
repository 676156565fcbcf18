// out[m,n] = sum_k x[m,k] * w[n,k] for a few rows of x (decode steps): a weight-streaming product in bfloat16 with
// 32-bit accumulation. The work is reading w once at memory speed, so the roles of the operands are swapped: sixteen
// rows of w are the 16-row operand of mma.m16n8k16 and up to 32 rows of x are its 8-wide columns. A CTA owns sixteen
// rows of w; its eight warps split k among them, each streaming its slice from global memory straight into registers
// (16 bytes a thread, several loads in flight, no L1 allocation) and the warps' partial sums meet in shared memory in
// warp order. The k index inside a 32-wide step is permuted the same way for both operands (a thread takes eight
// consecutive k of a row of w and the same eight of a row of x), which a dot product does not notice.
// Each output column depends on its own row of x only, so a row's bits do not depend on what else is in the batch.
// The reference calls cuBLASLt for every product (kernels/src/gemm.cu:235); its definition is CpuOps.Gemm
// (src/Starlings.Roost.Ops/CpuOps.cs:395-437): TransposeB, alpha 1, no bias, 32-bit accumulation, one rounding.
#include "common.cuh"

namespace roost {

constexpr int kSkinnyWarps = 8;
constexpr int kSkinnyUnroll = 4;

__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_cached_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT, typename TOut>
__global__ void __launch_bounds__(kSkinnyWarps * 32)
    gemm_skinny_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, TOut* __restrict__ out, int M, int N, int K,
                       int64_t ldx, int64_t ldw, int64_t ldo) {
  __shared__ float red[kSkinnyWarps][16][NT * 8 + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int n0 = blockIdx.x * 16;
  const __nv_bfloat16* w_lo = w + (size_t)(n0 + g) * ldw + q * 8;
  const __nv_bfloat16* w_hi = w_lo + 8 * ldw;
  const __nv_bfloat16* x_row[NT];
  bool x_ok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    x_ok[nt] = nt * 8 + g < M;
    x_row[nt] = x + (size_t)(x_ok[nt] ? nt * 8 + g : 0) * ldx + q * 8;
  }
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

  const int steps = K / 32;
  const int s_begin = (int)((int64_t)warp * steps / kSkinnyWarps);
  const int s_end = (int)((int64_t)(warp + 1) * steps / kSkinnyWarps);

  // Two register buffers of kSkinnyUnroll steps each: the loads of the next group of steps are issued before the
  // products of the current group, so every thread always has a group of 16-byte loads in flight.
  uint4 wa[2][kSkinnyUnroll], wb[2][kSkinnyUnroll];
  auto load_group = [&](int buf, int s) {
#pragma unroll
    for (int u = 0; u < kSkinnyUnroll; ++u) {
      if (s + u < s_end) {
        wa[buf][u] = ld_stream_16(w_lo + (size_t)(s + u) * 32);
        wb[buf][u] = ld_stream_16(w_hi + (size_t)(s + u) * 32);
      }
    }
  };
  auto compute_group = [&](int buf, int s) {
#pragma unroll
    for (int u = 0; u < kSkinnyUnroll; ++u) {
      if (s + u < s_end) {
        uint4 xv[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          xv[nt] = make_uint4(0u, 0u, 0u, 0u);
          if (x_ok[nt]) xv[nt] = ld_cached_16(x_row[nt] + (size_t)(s + u) * 32);
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          mma_bf16_16816(acc[nt], wa[buf][u].x, wb[buf][u].x, wa[buf][u].y, wb[buf][u].y, xv[nt].x, xv[nt].y);
          mma_bf16_16816(acc[nt], wa[buf][u].z, wb[buf][u].z, wa[buf][u].w, wb[buf][u].w, xv[nt].z, xv[nt].w);
        }
      }
    }
  };
  load_group(0, s_begin);
  for (int s = s_begin; s < s_end; s += 2 * kSkinnyUnroll) {
    load_group(1, s + kSkinnyUnroll);
    compute_group(0, s);
    load_group(0, s + 2 * kSkinnyUnroll);
    compute_group(1, s + kSkinnyUnroll);
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    red[warp][g][nt * 8 + q * 2] = acc[nt][0];
    red[warp][g][nt * 8 + q * 2 + 1] = acc[nt][1];
    red[warp][g + 8][nt * 8 + q * 2] = acc[nt][2];
    red[warp][g + 8][nt * 8 + q * 2 + 1] = acc[nt][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 16 * M; idx += kSkinnyWarps * 32) {
    const int m = idx / 16, r = idx % 16;  // consecutive threads write consecutive n of one output row
    float v = 0.f;
#pragma unroll
    for (int ww = 0; ww < kSkinnyWarps; ++ww) v += red[ww][r][m];
    out[(size_t)m * ldo + n0 + r] = from_float<TOut>(v);
  }
}

template <int NT>
static int launch_skinny(const void* x, const void* w, void* out, int m, int n, int k, int64_t ldx, int64_t ldw, int64_t ldo,
                         int out_dtype, cudaStream_t s) {
  const dim3 grid(n / 16);
  if (out_dtype == ROOST_BF16) {
    gemm_skinny_kernel<NT, __nv_bfloat16><<<grid, kSkinnyWarps * 32, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                                                              (__nv_bfloat16*)out, m, n, k, ldx, ldw, ldo);
  } else {
    gemm_skinny_kernel<NT, float><<<grid, kSkinnyWarps * 32, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (float*)out, m, n,
                                                                      k, ldx, ldw, ldo);
  }
  return check_launch("gemm_skinny");
}

}  // namespace roost

using namespace roost;

extern "C" int roost_gemm_skinny_supported(int m, int n, int k, int64_t ldx, int64_t ldw) {
  return m >= 1 && m <= 32 && n % 16 == 0 && k % 32 == 0 && k >= 32 * kSkinnyWarps && ldx % 8 == 0 && ldw % 8 == 0;
}

extern "C" int roost_gemm_skinny(const void* x, const void* w, void* out, int m, int n, int k, int64_t ldx, int64_t ldw, int64_t ldo,
                                 int out_dtype, roost_stream_t stream) {
  ROOST_REQUIRE(out_dtype == ROOST_BF16 || out_dtype == ROOST_F32, "gemm_skinny: the output is bfloat16 (1) or float32 (0)");
  ROOST_REQUIRE(ldx >= k && ldw >= k && ldo >= n, "gemm_skinny: a leading dimension is smaller than its row");
  if (!roost_gemm_skinny_supported(m, n, k, ldx, ldw)) {
    return fail(ROOST_ERR_UNSUPPORTED, "gemm_skinny: needs 1 <= m <= 32, n a multiple of 16, k a multiple of 32 and at least 256, rows on 16-byte boundaries");
  }
  ROOST_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_skinny: x and w must start on 16-byte boundaries");
  cudaStream_t s = (cudaStream_t)stream;
  switch ((m + 7) / 8) {
    case 1: return launch_skinny<1>(x, w, out, m, n, k, ldx, ldw, ldo, out_dtype, s);
    case 2: return launch_skinny<2>(x, w, out, m, n, k, ldx, ldw, ldo, out_dtype, s);
    case 3: return launch_skinny<3>(x, w, out, m, n, k, ldx, ldw, ldo, out_dtype, s);
    default: return launch_skinny<4>(x, w, out, m, n, k, ldx, ldw, ldo, out_dtype, s);
  }
}
