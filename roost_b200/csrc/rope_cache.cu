// Per-head RMS norm of q and k, NeoX rotation, and the write of k and v into their page slots, in one pass
// over the projected qkv rows.
//
// What it must compute is the reference's unfused sequence QkNorm -> Rope -> CacheWrite in that order
// (src/Starlings.Roost.Ops/CpuOps.Fused.cs:51-97; parts at CpuOps.cs:65-85, :111-177, :515-554): the norm is
// over head_dim with one weight vector shared by the heads, values are not normed or rotated, a negative slot
// is skipped. The angle position * inv_freq[i] is formed in double and reduced to [-pi, pi] before the 32-bit
// sincosf, as the reference's device kernel does (kernels/src/m0_ops.cu:163,187-190), because a 32-bit angle
// loses the rotation at large positions. The page layout is [page][kv head][offset in page][head_dim].
#include "common.cuh"

namespace roost {

// One warp per (token, head slot); head slots are q heads, then k heads, then v heads.
template <typename T>
__global__ void qk_norm_rope_cache_kernel(const T* __restrict__ qkv, int64_t qkv_stride, T* __restrict__ q_out,
                                          T* __restrict__ k_pool, T* __restrict__ v_pool, const void* __restrict__ q_w,
                                          const void* __restrict__ k_w, const double* __restrict__ inv_freq,
                                          const int32_t* __restrict__ positions, const int32_t* __restrict__ slot_mapping,
                                          int q_heads, int kv_heads, int head_dim, int rotary_dim, float eps, int page_size,
                                          int64_t pool_pages, int slots_per_token, int wdtype) {
  const int lane = threadIdx.x & 31;
  const int slot_idx = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (slot_idx >= slots_per_token) return;
  const size_t t = blockIdx.x;
  const T* row = qkv + t * qkv_stride;

  int kind, head;  // 0 q, 1 k, 2 v
  if (slot_idx < q_heads) {
    kind = 0; head = slot_idx;
  } else if (slot_idx < q_heads + kv_heads) {
    kind = 1; head = slot_idx - q_heads;
  } else {
    kind = 2; head = slot_idx - q_heads - kv_heads;
  }
  const T* src = row + (size_t)slot_idx * head_dim;  // [q heads | k heads | v heads], each head_dim wide

  T* dst;
  if (kind == 0) {
    dst = q_out + (t * q_heads + head) * head_dim;
  } else {
    const int slot = slot_mapping[t];
    if (slot < 0) return;
    const int64_t page = slot / page_size;
    const int off = slot % page_size;
    if (page >= pool_pages) return;  // never write beyond the pool
    T* pool = kind == 1 ? k_pool : v_pool;
    dst = pool + ((page * kv_heads + head) * page_size + off) * head_dim;
  }

  if (kind == 2) {
    for (int i = lane; i < head_dim; i += 32) dst[i] = src[i];
    return;
  }

  const void* w = kind == 0 ? q_w : k_w;
  float inv = 1.0f;
  if (w != nullptr) {
    float ss = 0.f;
    for (int i = lane; i < head_dim; i += 32) {
      const float v = to_float(src[i]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)head_dim + eps);
  }
  const int half = rotary_dim / 2;
  const double pos = (double)positions[t];
  // rotated pairs (i, i + half)
  for (int i = lane; i < half; i += 32) {
    float x1 = to_float(src[i]);
    float x2 = to_float(src[i + half]);
    if (w != nullptr) {
      // the normed value stays in 32-bit until the rotation has used it: one rounding per output element
      x1 = x1 * inv * load_w(w, i, wdtype);
      x2 = x2 * inv * load_w(w, i + half, wdtype);
    }
    double ang = pos * inv_freq[i];
    ang -= 6.283185307179586476925286766559 * rint(ang * 0.15915494309189533576888376337251);
    float s, c;
    sincosf((float)ang, &s, &c);
    dst[i] = from_float<T>(x1 * c - x2 * s);
    dst[i + half] = from_float<T>(x2 * c + x1 * s);
  }
  // elements at and beyond rotary_dim are normed only
  for (int i = rotary_dim + lane; i < head_dim; i += 32) {
    float x = to_float(src[i]);
    if (w != nullptr) x = x * inv * load_w(w, i, wdtype);
    dst[i] = from_float<T>(x);
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_qk_norm_rope_cache(const void* qkv, int64_t qkv_stride, void* q_out, void* k_pool, void* v_pool,
                                        const void* q_w, const void* k_w, const double* inv_freq,
                                        const int32_t* positions, const int32_t* slot_mapping, int tokens, int q_heads,
                                        int kv_heads, int head_dim, int rotary_dim, float eps, int page_size,
                                        int64_t pool_pages, int write_kv, int dtype, int wdtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads >= 0 && head_dim > 0, "qk_norm_rope_cache: sizes must be positive");
  ROOST_REQUIRE(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
                "qk_norm_rope_cache: rotary_dim must be even and at most head_dim");
  ROOST_REQUIRE(rotary_dim == 0 || inv_freq != nullptr, "qk_norm_rope_cache: inv_freq is null");
  ROOST_REQUIRE(rotary_dim == 0 || positions != nullptr, "qk_norm_rope_cache: positions is null");
  ROOST_REQUIRE((q_w == nullptr) == (k_w == nullptr) || !write_kv, "qk_norm_rope_cache: q and k norm weights come together");
  if (write_kv) {
    ROOST_REQUIRE(k_pool && v_pool && slot_mapping && page_size > 0 && pool_pages > 0 && kv_heads > 0,
                  "qk_norm_rope_cache: the cache pools, the slot mapping and the page geometry are needed to write");
  }
  if (tokens == 0) return ROOST_OK;
  const int slots = q_heads + (write_kv ? 2 * kv_heads : 0);
  const int warps = 4;
  dim3 grid(tokens, (slots + warps - 1) / warps);
  if (grid.y > 65535) return fail(ROOST_ERR_UNSUPPORTED, "qk_norm_rope_cache: more than 262140 head slots per token");
  ROOST_DISPATCH_DTYPE(dtype, T,
                       qk_norm_rope_cache_kernel<T><<<grid, warps * 32, 0, (cudaStream_t)stream>>>(
                           (const T*)qkv, qkv_stride, (T*)q_out, (T*)k_pool, (T*)v_pool, q_w, k_w, inv_freq, positions,
                           slot_mapping, q_heads, kv_heads, head_dim, rotary_dim, eps, page_size, pool_pages, slots, wdtype));
  return check_launch("qk_norm_rope_cache");
}
