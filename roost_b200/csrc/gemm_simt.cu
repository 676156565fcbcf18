// out[m,n] = sum_k a[m,k] * w[n,k] with plain 32-bit FFMA: the matrix product of the float32 model (no tensor
// cores, no reduced-precision mode), also usable with bfloat16 operands for checks. Every output element sums
// over k in increasing order in one thread, so its bits do not depend on m's or n's extent or on the tile a
// row falls in. Definition: src/Starlings.Roost.Ops/CpuOps.cs:395-437 (TransposeB, Alpha 1, no bias).
#include "common.cuh"

namespace roost {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TIn* __restrict__ a, const TIn* __restrict__ w,
                                                       TOut* __restrict__ out, int M, int N, int K, int64_t lda,
                                                       int64_t ldw, int64_t ldo) {
  __shared__ float as[BK][BM + 1];
  __shared__ float ws[BK][BN + 1];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      const int row = idx >> 4, col = idx & 15;
      const int k = k0 + col;
      const int m = m0 + row, n = n0 + row;
      as[col][row] = (m < M && k < K) ? to_float(a[(int64_t)m * lda + k]) : 0.f;
      ws[col][row] = (n < N && k < K) ? to_float(w[(int64_t)n * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = as[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[(int64_t)m * ldo + n] = from_float<TOut>(acc[i][j]);
    }
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_gemm_simt(const void* a, const void* w, void* out, int m, int n, int k, int64_t lda, int64_t ldw,
                               int64_t ldo, int in_dtype, int out_dtype, roost_stream_t stream) {
  ROOST_REQUIRE(m >= 0 && n > 0 && k > 0, "gemm: m, n and k must be positive");
  ROOST_REQUIRE(lda >= k && ldw >= k && ldo >= n, "gemm: a leading dimension is smaller than its row");
  if (m == 0) return ROOST_OK;
  dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
  if (grid.y > 65535) return fail(ROOST_ERR_UNSUPPORTED, "gemm: more than 4194240 rows in one product");
  cudaStream_t s = (cudaStream_t)stream;
  if (in_dtype == ROOST_F32 && out_dtype == ROOST_F32) {
    gemm_simt_kernel<float, float><<<grid, 256, 0, s>>>((const float*)a, (const float*)w, (float*)out, m, n, k, lda, ldw, ldo);
  } else if (in_dtype == ROOST_BF16 && out_dtype == ROOST_BF16) {
    gemm_simt_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)w,
                                                                       (__nv_bfloat16*)out, m, n, k, lda, ldw, ldo);
  } else if (in_dtype == ROOST_BF16 && out_dtype == ROOST_F32) {
    gemm_simt_kernel<__nv_bfloat16, float><<<grid, 256, 0, s>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (float*)out,
                                                               m, n, k, lda, ldw, ldo);
  } else {
    return fail(ROOST_ERR_INVALID, "gemm: dtype codes must be (0,0), (1,1) or (1,0) for (in, out)");
  }
  return check_launch("gemm_simt");
}
