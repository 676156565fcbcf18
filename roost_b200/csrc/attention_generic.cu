// Causal grouped-query attention over the paged cache in 32-bit arithmetic: the path of the float32 model and
// of head sizes no tensor-core kernel serves.
//
// Definition: src/Starlings.Roost.Ops/CpuOps.cs:181-298. A query at absolute position p sees keys
// max(0, p - window + 1) .. p (no window: from 0); query head h reads key/value head h / (q_heads / kv_heads);
// score = q.k * scale; softmax with a running maximum; output = sum p_j v_j / sum p_j.
//
// One block per (query token, key/value head, group of 4 query heads); each warp owns one query head. Keys are
// visited in tiles of 32 at absolute positions that are multiples of 32, a lane per key, so the order of every
// sum depends on the query's position alone: the same token gives the same bits whether it arrives in a whole
// prompt, a portion or a single decode step, and whatever else is in the batch.
#include "common.cuh"

namespace roost {

constexpr int kTile = 32;
constexpr int kWarps = 4;
constexpr int kMaxHeadDim = 512;

template <typename T>
__global__ void paged_attention_generic_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ k_pool,
                                               const T* __restrict__ v_pool, const int32_t* __restrict__ positions,
                                               const int32_t* __restrict__ token_row, const int32_t* __restrict__ kv_indptr,
                                               const int32_t* __restrict__ kv_indices, int q_heads, int kv_heads, int head_dim,
                                               int page_size, float scale, int window) {
  extern __shared__ float smem[];
  const int d = head_dim;
  const int dk = d + 1;                       // padded key rows: a lane per key reads without bank conflicts
  float* ks = smem;                           // [kTile][d + 1]
  float* vs = ks + kTile * dk;                // [kTile][d]
  float* qs = vs + kTile * d;                 // [kWarps][d]
  float* ps = qs + kWarps * d;                // [kWarps][kTile]

  const int t = blockIdx.x;
  const int kvh = blockIdx.y;
  const int group = q_heads / kv_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.z * kWarps + warp;   // head within the group
  const bool active = g < group;
  const int h = kvh * group + g;

  const int pos = positions[t];
  const int b = token_row[t];
  const int32_t* pages = kv_indices + kv_indptr[b];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;

  if (active) {
    const T* qv = q + ((size_t)t * q_heads + h) * d;
    for (int i = lane; i < d; i += 32) qs[warp * d + i] = to_float(qv[i]);
  }

  float m = -INFINITY, l = 0.f;
  float o[kMaxHeadDim / 32];
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) o[i] = 0.f;

  for (int j0 = (lo / kTile) * kTile; j0 <= pos; j0 += kTile) {
    __syncthreads();  // the previous tile has been consumed (and qs is written, the first time)
    // load the tile: keys j0 .. j0+31 that are visible
    for (int r = warp; r < kTile; r += kWarps) {
      const int j = j0 + r;
      if (j >= lo && j <= pos) {
        const int page = pages[j / page_size];
        const size_t base = (((size_t)page * kv_heads + kvh) * page_size + (j % page_size)) * d;
        for (int i = lane; i < d; i += 32) {
          ks[r * dk + i] = to_float(k_pool[base + i]);
          vs[r * d + i] = to_float(v_pool[base + i]);
        }
      } else {
        for (int i = lane; i < d; i += 32) {
          ks[r * dk + i] = 0.f;
          vs[r * d + i] = 0.f;
        }
      }
    }
    __syncthreads();
    if (active) {
      const int j = j0 + lane;
      const bool vis = j >= lo && j <= pos;
      float s = 0.f;
      const float* kr = ks + lane * dk;
      const float* qr = qs + warp * d;
      for (int i = 0; i < d; ++i) s = fmaf(qr[i], kr[i], s);
      s = vis ? s * scale : -INFINITY;
      const float m_new = fmaxf(m, warp_max(s));  // the tile holds at least one visible key
      const float p = vis ? expf(s - m_new) : 0.f;
      const float corr = expf(m - m_new);          // 0 on the first tile (m = -inf)
      l = l * corr + warp_sum(p);
      m = m_new;
      ps[warp * kTile + lane] = p;
      __syncwarp();
      const float* pr = ps + warp * kTile;
#pragma unroll
      for (int c = 0; c < kMaxHeadDim / 32; ++c) {
        const int i = c * 32 + lane;
        if (i < d) {
          float acc = o[c] * corr;
          for (int r = 0; r < kTile; ++r) acc = fmaf(pr[r], vs[r * d + i], acc);
          o[c] = acc;
        }
      }
      __syncwarp();
    }
  }
  if (active) {
    T* ov = out + ((size_t)t * q_heads + h) * d;
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int c = 0; c < kMaxHeadDim / 32; ++c) {
      const int i = c * 32 + lane;
      if (i < d) ov[i] = from_float<T>(o[c] * inv);
    }
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_paged_attention_generic(const void* q, void* out, const void* k_pool, const void* v_pool,
                                             const int32_t* positions, const int32_t* token_row,
                                             const int32_t* kv_indptr, const int32_t* kv_indices, int tokens,
                                             int q_heads, int kv_heads, int head_dim, int page_size, float scale,
                                             int window, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && head_dim > 0 && page_size > 0,
                "paged_attention: sizes must be positive");
  ROOST_REQUIRE(q_heads % kv_heads == 0, "paged_attention: q_heads must be a multiple of kv_heads");
  if (head_dim > kMaxHeadDim) return fail(ROOST_ERR_UNSUPPORTED, "paged_attention: head_dim beyond 512");
  if (kv_heads > 65535) return fail(ROOST_ERR_UNSUPPORTED, "paged_attention: more than 65535 key/value heads");
  if (tokens == 0) return ROOST_OK;
  const int group = q_heads / kv_heads;
  dim3 grid(tokens, kv_heads, (group + kWarps - 1) / kWarps);
  const size_t smem = ((size_t)kTile * (head_dim + 1) + (size_t)kTile * head_dim + (size_t)kWarps * head_dim + kWarps * kTile) * sizeof(float);
  ROOST_DISPATCH_DTYPE(dtype, T, {
    auto kernel = paged_attention_generic_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kernel<<<grid, kWarps * 32, smem, (cudaStream_t)stream>>>((const T*)q, (T*)out, (const T*)k_pool, (const T*)v_pool,
                                                              positions, token_row, kv_indptr, kv_indices, q_heads, kv_heads,
                                                              head_dim, page_size, scale, window);
  });
  return check_launch("paged_attention_generic");
}
