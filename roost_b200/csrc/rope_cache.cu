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
                                          const float2* __restrict__ step_table, int q_heads, int kv_heads, int head_dim, int rotary_dim,
                                          float eps, int page_size, int64_t pool_pages, int slots_per_token, int wdtype, bool vector_ok) {
  extern __shared__ float2 cos_sin[];  // [rotary_dim / 2]
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  pdl_launch_dependents(3);
  pdl_wait(3);
  const size_t t = blockIdx.x;
  const T* row = qkv + t * qkv_stride;
  const int half = rotary_dim / 2;
  const double pos = half > 0 && step_table == nullptr ? (double)positions[t] : 0.0;
  auto rotation = [&](int i) {  // (cos, sin) of the pair i: from the step's table, or computed here
    if (step_table != nullptr) return step_table[t * half + i];
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

// bfloat16, every element rotated, a head of 64, 128 or 256 elements, 16-byte aligned rows, more than a few tokens.
// A lane owns four elements of the head's first half and the four that pair with them in the second half (two 8-byte
// accesses), so a rotation needs no exchange between lanes. D / 8 lanes serve a part of a token: some of its head slots
// in turn, four loaded ahead; the sum of squares is reduced over the part's lanes. The part's cosines and sines (read from
// the step's table, else computed in the reference's 64-bit form), the norm weights and the token's place in the cache
// stay in registers, nothing goes through shared memory and no thread waits for another. A token has as many parts as
// fill the device's thread slots once: measured on a B200 against a block that takes whole tokens in turn with their
// table in shared memory, 15.3 against 15.2 us at 2,048 tokens of 32 + 8 + 8 heads, 5.6 against 6.6 at 512, 43 against
// 53 at 8,192; two to six times as many parts were slower.
template <int D>
__global__ void __launch_bounds__(256, 4) qk_norm_rope_cache_parts_kernel(
    const __nv_bfloat16* __restrict__ qkv, int64_t qkv_stride, __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pool,
    __nv_bfloat16* __restrict__ v_pool, const void* __restrict__ q_w, const void* __restrict__ k_w, const double* __restrict__ inv_freq,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ slot_mapping, const float2* __restrict__ step_table, int tokens,
    int parts, int slots_per_part, int q_heads, int kv_heads, float eps, int page_size, int page_shift, int64_t pool_pages,
    int slots_per_token, int wdtype) {
  constexpr int kLanes = D / 8;          // lanes of a part
  constexpr int kHalf = D / 2;
  constexpr int kAhead = 4;
  const int lane = threadIdx.x & 31;
  const int sub = lane / kLanes, c = lane % kLanes;   // which part of the warp's; which four pairs of a head
  const unsigned part_lanes = kLanes == 32 ? 0xffffffffu : ((1u << kLanes) - 1u) << (sub * kLanes);
  float wq_lo[4], wq_hi[4], wk_lo[4], wk_hi[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    wq_lo[e] = q_w ? load_w(q_w, 4 * c + e, wdtype) : 1.0f;
    wq_hi[e] = q_w ? load_w(q_w, kHalf + 4 * c + e, wdtype) : 1.0f;
    wk_lo[e] = k_w ? load_w(k_w, 4 * c + e, wdtype) : 1.0f;
    wk_hi[e] = k_w ? load_w(k_w, kHalf + 4 * c + e, wdtype) : 1.0f;
  }
  const bool normed = q_w != nullptr;
  const int64_t group = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / kLanes;
  const int t = (int)(group / parts), part = (int)(group - (int64_t)t * parts);
  pdl_launch_dependents(3);
  pdl_wait(3);
  if (t >= tokens) return;   // a whole part: its lanes leave together
  float cs[4], sn[4];
  if (step_table != nullptr) {
    const float4 r0 = *reinterpret_cast<const float4*>(step_table + (size_t)t * kHalf + 4 * c);
    const float4 r1 = *reinterpret_cast<const float4*>(step_table + (size_t)t * kHalf + 4 * c + 2);
    cs[0] = r0.x; sn[0] = r0.y; cs[1] = r0.z; sn[1] = r0.w;
    cs[2] = r1.x; sn[2] = r1.y; cs[3] = r1.z; sn[3] = r1.w;
  } else {
    const double pos = (double)positions[t];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      double ang = pos * inv_freq[4 * c + e];
      ang -= 6.283185307179586476925286766559 * rint(ang * 0.15915494309189533576888376337251);
      sincosf((float)ang, &sn[e], &cs[e]);
    }
  }
  auto unpack = [](const uint2 u, float (&v)[4]) {
    v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xffff0000u);
    v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xffff0000u);
  };
  auto store_half = [](__nv_bfloat16* p, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
  };
  const int slot = slot_mapping ? slot_mapping[t] : -1;
  const unsigned page = slot < 0 ? 0u : (page_shift >= 0 ? (unsigned)slot >> page_shift : (unsigned)slot / (unsigned)page_size);
  const unsigned off = slot < 0 ? 0u : (unsigned)slot - page * (unsigned)page_size;
  const bool cache_ok = slot >= 0 && (int64_t)page < pool_pages;
  const __nv_bfloat16* row = qkv + (size_t)t * qkv_stride + 4 * c;
  const int s_end = min(slots_per_token, (part + 1) * slots_per_part);
  for (int s0 = part * slots_per_part; s0 < s_end; s0 += kAhead) {
    uint2 raw_lo[kAhead], raw_hi[kAhead];
#pragma unroll
    for (int p = 0; p < kAhead; ++p) {
      if (s0 + p < s_end) {
        const __nv_bfloat16* src = row + (size_t)(s0 + p) * D;
        raw_lo[p] = *reinterpret_cast<const uint2*>(src);
        raw_hi[p] = *reinterpret_cast<const uint2*>(src + kHalf);
      }
    }
#pragma unroll
    for (int p = 0; p < kAhead; ++p) {
      const int slot_idx = s0 + p;
      if (slot_idx >= s_end) break;
      __nv_bfloat16* dst;
      if (slot_idx >= q_heads + kv_heads) {   // a value head: copied as it is
        if (!cache_ok) continue;
        dst = v_pool + (((size_t)page * kv_heads + (slot_idx - q_heads - kv_heads)) * page_size + off) * D + 4 * c;
        *reinterpret_cast<uint2*>(dst) = raw_lo[p];
        *reinterpret_cast<uint2*>(dst + kHalf) = raw_hi[p];
        continue;
      }
      float lo[4], hi[4];
      unpack(raw_lo[p], lo);
      unpack(raw_hi[p], hi);
      const bool is_q = slot_idx < q_heads;
      if (!is_q && !cache_ok) continue;
      float inv = 1.0f;
      if (normed) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) ss += lo[e] * lo[e] + hi[e] * hi[e];
#pragma unroll
        for (int o = kLanes / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(part_lanes, ss, o, kLanes);
        inv = 1.0f / sqrtf(ss / (float)D + eps);
      }
      float o_lo[4], o_hi[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float x1 = lo[e] * inv * (is_q ? wq_lo[e] : wk_lo[e]), x2 = hi[e] * inv * (is_q ? wq_hi[e] : wk_hi[e]);
        o_lo[e] = x1 * cs[e] - x2 * sn[e];
        o_hi[e] = x2 * cs[e] + x1 * sn[e];
      }
      dst = is_q ? q_out + ((size_t)t * q_heads + slot_idx) * D + 4 * c
                 : k_pool + (((size_t)page * kv_heads + (slot_idx - q_heads)) * page_size + off) * D + 4 * c;
      store_half(dst, o_lo);
      store_half(dst + kHalf, o_hi);
    }
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_qk_norm_rope_cache(const void* qkv, int64_t qkv_stride, void* q_out, void* k_pool, void* v_pool,
                                        const void* q_w, const void* k_w, const double* inv_freq,
                                        const int32_t* positions, const int32_t* slot_mapping, const float* cos_sin, int tokens,
                                        int q_heads, int kv_heads, int head_dim, int rotary_dim, float eps, int page_size,
                                        int64_t pool_pages, int write_kv, int dtype, int wdtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads >= 0 && head_dim > 0, "qk_norm_rope_cache: sizes must be positive");
  ROOST_REQUIRE(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
                "qk_norm_rope_cache: rotary_dim must be even and at most head_dim");
  ROOST_REQUIRE(rotary_dim == 0 || inv_freq != nullptr, "qk_norm_rope_cache: inv_freq is null");
  ROOST_REQUIRE(rotary_dim == 0 || positions != nullptr, "qk_norm_rope_cache: positions is null");
  ROOST_REQUIRE(cos_sin == nullptr || (uintptr_t)cos_sin % 16 == 0, "qk_norm_rope_cache: the table of cosines and sines must start on a 16-byte boundary");
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
  // bfloat16 heads of 64, 128 or 256 elements, all rotated, from 64 tokens on: the vector kernel
  if (dtype == ROOST_BF16 && vector_ok && rotary_dim == head_dim && tokens >= 64 && (head_dim == 64 || head_dim == 128 || head_dim == 256) &&
      (q_w == nullptr) == (k_w == nullptr)) {
    // as many parts a token as fill the device's thread slots once, at most one a head slot
    const int lanes = head_dim / 8;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int64_t parts = (int64_t)sms * 1024 / ((int64_t)tokens * lanes);
    parts = parts < 1 ? 1 : (parts > slots ? slots : parts);
    const int per_part = (int)((slots + parts - 1) / parts);
    parts = (slots + per_part - 1) / per_part;
    const int64_t blocks = ((int64_t)tokens * parts * lanes + 255) / 256;
    if (blocks > 0x7fffffff) return fail(ROOST_ERR_UNSUPPORTED, "qk_norm_rope_cache: more blocks than a grid holds");
    int page_shift = -1;   // pages of a power of two of tokens: a shift instead of a division
    for (int b = 0; b < 31 && page_size > 0; ++b)
      if (page_size == (1 << b)) page_shift = b;
    auto launch = [&](auto kernel) {
      launch_kernel(kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)qkv, qkv_stride,
                    (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, q_w, k_w, inv_freq, positions, slot_mapping,
                    (const float2*)cos_sin, tokens, (int)parts, per_part, q_heads, kv_heads, eps, page_size, page_shift, pool_pages, slots,
                    wdtype);
    };
    if (head_dim == 64) launch(qk_norm_rope_cache_parts_kernel<64>);
    else if (head_dim == 128) launch(qk_norm_rope_cache_parts_kernel<128>);
    else launch(qk_norm_rope_cache_parts_kernel<256>);
    return check_launch("qk_norm_rope_cache");
  }
  ROOST_DISPATCH_DTYPE(dtype, T, {
    auto kernel = many ? qk_norm_rope_cache_kernel<T, true> : qk_norm_rope_cache_kernel<T, false>;
    launch_kernel(kernel, grid, dim3(warps * 32), many ? table_bytes : 0, (cudaStream_t)stream, (const T*)qkv, qkv_stride, (T*)q_out,
                  (T*)k_pool, (T*)v_pool, q_w, k_w, inv_freq, positions, slot_mapping, (const float2*)cos_sin, q_heads, kv_heads, head_dim,
                  rotary_dim, eps, page_size, pool_pages, slots, wdtype, vector_ok);
  });
  return check_launch("qk_norm_rope_cache");
}

namespace roost {
__global__ void rope_table_kernel(const int32_t* __restrict__ positions, const double* __restrict__ inv_freq, int tokens, int half,
                                  float2* __restrict__ cos_sin) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t n = (int64_t)tokens * half;
  for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (int64_t)gridDim.x * blockDim.x) {
    double ang = (double)positions[j / half] * inv_freq[j % half];
    ang -= 6.283185307179586476925286766559 * rint(ang * 0.15915494309189533576888376337251);
    float sn, cs;
    sincosf((float)ang, &sn, &cs);
    cos_sin[j] = make_float2(cs, sn);
  }
}
}  // namespace roost

extern "C" int roost_rope_table(const int32_t* positions, const double* inv_freq, int tokens, int half, float* cos_sin,
                                roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && half > 0, "rope_table: tokens and half must be positive");
  ROOST_REQUIRE(positions && inv_freq && cos_sin, "rope_table: positions, inv_freq and the table are needed");
  if (tokens == 0) return ROOST_OK;
  const int64_t n = (int64_t)tokens * half;
  const int blocks = (int)((n + 127) / 128 > 4096 ? 4096 : (n + 127) / 128);
  launch_kernel(rope_table_kernel, dim3(blocks), dim3(128), 0, (cudaStream_t)stream, positions, inv_freq, tokens, half,
                reinterpret_cast<float2*>(cos_sin));
  return check_launch("rope_table");
}

ROOST_TRACE_TU(rope_cache)
