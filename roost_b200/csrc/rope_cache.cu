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

__device__ __forceinline__ void load2(const float* p, float (&v)[2]) {
  const float2 t = *reinterpret_cast<const float2*>(p);
  v[0] = t.x; v[1] = t.y;
}
__device__ __forceinline__ void load2(const __nv_bfloat16* p, float (&v)[2]) {
  const __nv_bfloat162 t = *reinterpret_cast<const __nv_bfloat162*>(p);
  v[0] = __low2float(t); v[1] = __high2float(t);
}
__device__ __forceinline__ void store2(float* p, const float (&v)[2]) { *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]); }
__device__ __forceinline__ void store2(__nv_bfloat16* p, const float (&v)[2]) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
}

// One block per token (and, for few tokens, per group of head slots); a warp takes head slots in turn. Head slots are
// q heads, then k heads, then v heads. The rotation's cosines and sines depend on the token's position only: with TABLE
// the block computes them once into shared memory and every head of the token uses them (many tokens: the arithmetic
// is the cost); without, every warp computes its own while its loads are in flight (few tokens: the latency is). vector_ok: every head row of qkv, q_out
// and the pools starts on a 16-byte boundary (head_dim a multiple of 8 elements, aligned bases and stride).
template <typename T, bool TABLE>
__global__ void qk_norm_rope_cache_kernel(const T* __restrict__ qkv, int64_t qkv_stride, T* __restrict__ q_out,
                                          T* __restrict__ k_pool, T* __restrict__ v_pool, const void* __restrict__ q_w,
                                          const void* __restrict__ k_w, const double* __restrict__ inv_freq,
                                          const int32_t* __restrict__ positions, const int32_t* __restrict__ slot_mapping,
                                          int q_heads, int kv_heads, int head_dim, int rotary_dim, float eps, int page_size,
                                          int64_t pool_pages, int slots_per_token, int wdtype, bool vector_ok) {
  extern __shared__ float2 cos_sin[];  // [rotary_dim / 2]
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  pdl_launch_dependents(3);
  pdl_wait(3);
  const size_t t = blockIdx.x;
  const T* row = qkv + t * qkv_stride;
  const int half = rotary_dim / 2;
  const double pos = half > 0 ? (double)positions[t] : 0.0;
  auto rotation = [&](int i) {  // (cos, sin) of the pair i
    double ang = pos * inv_freq[i];
    ang -= 6.283185307179586476925286766559 * rint(ang * 0.15915494309189533576888376337251);
    float sn, cs;
    sincosf((float)ang, &sn, &cs);
    return make_float2(cs, sn);
  };
  if (TABLE && half > 0) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) cos_sin[i] = rotation(i);
    __syncthreads();
  }

  // Many tokens of bfloat16 with every element rotated and a head of 64, 128 or 256: a lane owns eight neighbouring
  // elements (one 16-byte access) of a head slot, so a warp serves 32 / (head_dim / 8) slots at a time; the lane that
  // holds the other element of each of its pairs is head_dim / 16 lanes away, and the sum of squares is reduced over
  // the slot's lanes only. A fifth of the instructions of the element-by-element form below.
  if constexpr (TABLE && sizeof(T) == 2) {
    if (vector_ok && rotary_dim == head_dim && (head_dim == 64 || head_dim == 128 || head_dim == 256)) {
      const int lanes_per_slot = head_dim / 8, slots_per_pass = 32 / lanes_per_slot;
      const int sub = lane / lanes_per_slot, c = lane % lanes_per_slot;  // which slot of the pass, which chunk of its head
      const int pair_lanes = lanes_per_slot / 2;                        // the lane that holds the pairs' other elements: lane ^ pair_lanes
      const bool second = c >= pair_lanes;                              // this lane's elements are the x2 of their pairs
      const int i0 = (c % pair_lanes) * 8;                              // first pair index of the lane
      float wq[8], wk[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        wq[e] = q_w ? load_w(q_w, c * 8 + e, wdtype) : 1.0f;
        wk[e] = k_w ? load_w(k_w, c * 8 + e, wdtype) : 1.0f;
      }
      float cs[8], sn[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float2 r = cos_sin[i0 + e];
        cs[e] = r.x;
        sn[e] = second ? r.y : -r.y;  // x1' = x1 c - x2 s; x2' = x2 c + x1 s: own * c + other * (-+s)
      }
      const int slot = slot_mapping ? slot_mapping[t] : -1;
      const int64_t page = slot >= 0 ? slot / page_size : 0;
      const int off = slot >= 0 ? slot % page_size : 0;
      const bool cache_ok = slot >= 0 && page < pool_pages;
      const int first_warp_slot = (blockIdx.y * warps + (threadIdx.x >> 5)) * slots_per_pass;
      const int pass_stride = gridDim.y * warps * slots_per_pass;
      float x_next[8];
      auto fetch = [&](int base) {  // the lane's eight elements of the pass that starts at slot `base`
        if (base + sub < slots_per_token) {
          Vec<T>::load(row + (size_t)(base + sub) * head_dim + c * 8, x_next);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) x_next[e] = 0.f;
        }
      };
      fetch(first_warp_slot);
      for (int base = first_warp_slot; base < slots_per_token; base += pass_stride) {
        const int slot_idx = base + sub;
        const bool live = slot_idx < slots_per_token;
        int kind = 0, head = 0;
        if (live) {
          if (slot_idx < q_heads) {
            kind = 0; head = slot_idx;
          } else if (slot_idx < q_heads + kv_heads) {
            kind = 1; head = slot_idx - q_heads;
          } else {
            kind = 2; head = slot_idx - q_heads - kv_heads;
          }
        }
        float x[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = x_next[e];
        fetch(base + pass_stride);  // the next pass's elements travel while this pass is computed
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
        for (int o = lanes_per_slot / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const void* w = kind == 0 ? q_w : k_w;
        const float inv = (kind != 2 && w != nullptr) ? 1.0f / sqrtf(ss / (float)head_dim + eps) : 1.0f;
        float y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = kind == 2 ? x[e] : x[e] * inv * (kind == 0 ? wq[e] : wk[e]);
        float out[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float other = __shfl_xor_sync(0xffffffffu, y[e], pair_lanes);
          out[e] = kind == 2 ? y[e] : y[e] * cs[e] + other * sn[e];
        }
        if (!live) continue;
        T* dst;
        if (kind == 0) {
          dst = q_out + (t * q_heads + head) * head_dim;
        } else {
          if (!cache_ok) continue;  // a skipped token, or a slot beyond the pool: never written
          dst = (kind == 1 ? k_pool : v_pool) + ((page * kv_heads + head) * page_size + off) * head_dim;
        }
        Vec<T>::store(dst + c * 8, out);
      }
      return;
    }
  }

  for (int slot_idx = blockIdx.y * warps + (threadIdx.x >> 5); slot_idx < slots_per_token; slot_idx += gridDim.y * warps) {
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
      if (slot < 0) continue;
      const int64_t page = slot / page_size;
      const int off = slot % page_size;
      if (page >= pool_pages) continue;  // never write beyond the pool
      T* pool = kind == 1 ? k_pool : v_pool;
      dst = pool + ((page * kv_heads + head) * page_size + off) * head_dim;
    }

    if (kind == 2) {
      if (vector_ok) {
        constexpr int N = 16 / sizeof(T);
        for (int i = lane * N; i < head_dim; i += 32 * N) *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
      } else {
        for (int i = lane; i < head_dim; i += 32) dst[i] = src[i];
      }
      continue;
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
    // rotated pairs (i, i + half); two neighbouring pairs at a time when the layout allows 2-element accesses
    if (vector_ok && (half & 1) == 0) {
      for (int i = lane * 2; i < half; i += 64) {
        float a[2], b[2];
        load2(src + i, a);
        load2(src + i + half, b);
        float o1[2], o2[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float x1 = a[e], x2 = b[e];
          if (w != nullptr) {
            x1 = x1 * inv * load_w(w, i + e, wdtype);
            x2 = x2 * inv * load_w(w, i + e + half, wdtype);
          }
          const float2 r = TABLE ? cos_sin[i + e] : rotation(i + e);
          o1[e] = x1 * r.x - x2 * r.y;
          o2[e] = x2 * r.x + x1 * r.y;
        }
        store2(dst + i, o1);
        store2(dst + i + half, o2);
      }
    } else {
      for (int i = lane; i < half; i += 32) {
        float x1 = to_float(src[i]);
        float x2 = to_float(src[i + half]);
        if (w != nullptr) {
          // the normed value stays in 32-bit until the rotation has used it: one rounding per output element
          x1 = x1 * inv * load_w(w, i, wdtype);
          x2 = x2 * inv * load_w(w, i + half, wdtype);
        }
        const float2 r = TABLE ? cos_sin[i] : rotation(i);
        dst[i] = from_float<T>(x1 * r.x - x2 * r.y);
        dst[i + half] = from_float<T>(x2 * r.x + x1 * r.y);
      }
    }
    // elements at and beyond rotary_dim are normed only
    for (int i = rotary_dim + lane; i < head_dim; i += 32) {
      float x = to_float(src[i]);
      if (w != nullptr) x = x * inv * load_w(w, i, wdtype);
      dst[i] = from_float<T>(x);
    }
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
  // many tokens: one block of eight warps a token, the rotation table computed once a token; few tokens: four head
  // slots a block, so that a decode step still spreads over the device
  const bool many = tokens >= 512;
  const int warps = many ? 8 : 4;
  dim3 grid(tokens, many ? 1 : (slots + warps - 1) / warps);
  if (grid.y > 65535) return fail(ROOST_ERR_UNSUPPORTED, "qk_norm_rope_cache: more than 262140 head slots per token");
  const size_t table_bytes = (size_t)(rotary_dim / 2) * sizeof(float2);
  if (table_bytes > 48 * 1024) return fail(ROOST_ERR_UNSUPPORTED, "qk_norm_rope_cache: a rotary width beyond 12288");
  const size_t esize = dtype == ROOST_F32 ? 4 : 2;
  const bool vector_ok = (head_dim * esize) % 16 == 0 && (qkv_stride * esize) % 16 == 0 && (uintptr_t)qkv % 16 == 0 &&
                         (uintptr_t)q_out % 16 == 0 && (!write_kv || ((uintptr_t)k_pool % 16 == 0 && (uintptr_t)v_pool % 16 == 0));
  ROOST_DISPATCH_DTYPE(dtype, T, {
    auto kernel = many ? qk_norm_rope_cache_kernel<T, true> : qk_norm_rope_cache_kernel<T, false>;
    launch_kernel(kernel, grid, dim3(warps * 32), many ? table_bytes : 0, (cudaStream_t)stream, (const T*)qkv, qkv_stride, (T*)q_out,
                  (T*)k_pool, (T*)v_pool, q_w, k_w, inv_freq, positions, slot_mapping, q_heads, kv_heads, head_dim, rotary_dim, eps,
                  page_size, pool_pages, slots, wdtype, vector_ok);
  });
  return check_launch("qk_norm_rope_cache");
}

ROOST_TRACE_TU(rope_cache)
