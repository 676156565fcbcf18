// Greedy choice and temperature / top-k / top-p / min-p sampling on the device.
//
// The reference has no device sampler (src/Starlings.Roost.Worker/Eager/CudaOps.cs:293-332 falls back to the host);
// its definition of the result is CpuOps.Sample (src/Starlings.Roost.Ops/CpuOps.Sampling.cs:10-46, :279-370) and
// this kernel computes that result without sorting:
//   * NaN and -inf logits are removed; temperature <= 0 picks the highest logit, ties to the lowest index;
//   * p = softmax((z - max) / T); tokens are ordered by p descending, ties by lower index;
//   * top-k keeps the first k of that order, top-p the shortest prefix whose mass reaches top_p * (kept mass),
//     the crossing token included, min-p drops p < min_p * p_max;
//   * u = Philox4x32-10(counter = (offset lo, offset hi, 0, 0), key = (seed lo, seed hi)) word 0, top 24 bits
//     * 2^-24 (src/Starlings.Roost.Ops/CpuPhilox.cs:15-44); the chosen token is the first of the order whose
//     running kept mass exceeds u * (kept mass), the last kept token if rounding leaves none.
// A prefix of the order is the set {p > x} plus the first c tokens (by index) with p == x, so every step is a
// search for x over the bit patterns of p (non-negative floats order like their bits), 32 passes over the row
// with a block-wide sum each, and a count of ties. The sums run in a fixed order, so a row gives the same
// token in any batch and on any run. Sums differ in rounding from the reference's sequential sums over a
// sorted array: a draw within rounding of an interval's edge may fall to the neighbouring token.
#include "common.cuh"

namespace roost {

constexpr int kThreads = 1024;

__device__ __forceinline__ unsigned philox4x32_10(unsigned c0, unsigned c1, unsigned c2, unsigned c3, unsigned k0,
                                                  unsigned k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const uint32_t hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
    const uint32_t hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
    c0 = hi1 ^ c1 ^ k0;
    c1 = lo1;
    c2 = hi0 ^ c3 ^ k1;
    c3 = lo0;
    k0 += W0;
    k1 += W1;
  }
  return c0;
}

// Block-wide helpers. Every one is called by all 1024 threads under block-uniform control flow; each starts with a
// barrier so that the shared scratch of the previous call has been read by everyone.
__device__ __forceinline__ float block_sum_f(float v, float* sf) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) sf[warp] = v;
  __syncthreads();
  return warp_sum(sf[lane]);  // kThreads / 32 == 32 warps: every warp sums the same 32 values in the same order
}

__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ int block_sum_i(int v, int* si) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum_i(v);
  __syncthreads();
  if (lane == 0) si[warp] = v;
  __syncthreads();
  return warp_sum_i(si[lane]);
}

__device__ __forceinline__ bool better(float av, int ai, float cv, int ci) {
  if (ci < 0) return true;
  if (ai < 0) return false;
  return av > cv || (av == cv && ai < ci);
}

// Index of the maximum with ties to the lower index; NaN and (optionally) -inf never win; -1 when nothing
// qualifies. The maximum itself is left in sf[0] for the caller to read after the call.
__device__ __forceinline__ int block_argmax(const float* z, int n, bool skip_neg_inf, float* sf, int* si) {
  float bv = 0.f;
  int bi = -1;
  for (int v = threadIdx.x; v < n; v += kThreads) {
    const float x = z[v];
    if (x != x) continue;
    if (skip_neg_inf && x == -INFINITY) continue;
    if (bi < 0 || x > bv) {
      bv = x;
      bi = v;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (!better(bv, bi, ov, oi)) {
      bv = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) {
    sf[warp] = bv;
    si[warp] = bi;
  }
  __syncthreads();
  bv = sf[lane];
  bi = si[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (!better(bv, bi, ov, oi)) {
      bv = ov;
      bi = oi;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) sf[0] = bv;
  __syncthreads();
  return bi;
}

__global__ void __launch_bounds__(kThreads) argmax_kernel(const float* __restrict__ logits, long long stride, int vocab,
                                                         int* __restrict__ ids) {
  __shared__ float sf[32];
  __shared__ int si[32];
  const int r = blockIdx.x;
  const int best = block_argmax(logits + (size_t)r * stride, vocab, false, sf, si);
  if (threadIdx.x == 0) ids[r] = best;
}

// A row of a large vocabulary split over several blocks, so that one SM's bandwidth does not bound it: a block finds the
// best of its span and leaves it in part_v / part_i; the block that arrives last at the row's counter (after a fence)
// combines the spans in index order, writes the row's id and sets the counter back to zero for the next call.
__global__ void __launch_bounds__(kThreads) argmax_split_kernel(const float* __restrict__ logits, long long stride, int vocab,
                                                               int* __restrict__ ids, float* part_v, int* part_i, unsigned* counters) {
  __shared__ float sf[32];
  __shared__ int si[32];
  __shared__ int last;
  const int r = blockIdx.x, s = blockIdx.y, splits = gridDim.y;
  const int span = (((vocab + splits - 1) / splits) + 3) & ~3;
  const int lo = min(vocab, s * span), hi = min(vocab, lo + span);
  const int best = block_argmax(logits + (size_t)r * stride + lo, hi - lo, false, sf, si);
  if (threadIdx.x == 0) {
    part_v[r * splits + s] = sf[0];
    part_i[r * splits + s] = best < 0 ? -1 : best + lo;
    __threadfence();
    last = atomicAdd(&counters[r], 1u) == (unsigned)(splits - 1);
  }
  __syncthreads();
  if (!last || threadIdx.x >= 32) return;
  __threadfence();
  const int lane = threadIdx.x;
  float bv = lane < splits ? __ldcg(part_v + r * splits + lane) : 0.f;
  int bi = lane < splits ? __ldcg(part_i + r * splits + lane) : -1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (!better(bv, bi, ov, oi)) {
      bv = ov;
      bi = oi;
    }
  }
  if (lane == 0) {
    ids[r] = bi;
    counters[r] = 0u;
  }
}

// A kept prefix of the order is (xb, c): every key > xb, plus the first c tokens (by index) whose key == xb.
// Keys are the bit patterns of the probabilities; removed tokens hold -1 and are skipped.

// Mass of {key > xb}; the count of the same set is left in *count.
__device__ __forceinline__ float mass_gt(const float* p, int n, unsigned xb, int& count, float* sf, int* si) {
  float m = 0.f;
  int c = 0;
  for (int v = threadIdx.x; v < n; v += kThreads) {
    const float x = p[v];
    if (x >= 0.f && __float_as_uint(x) > xb) {
      m += x;
      ++c;
    }
  }
  count = block_sum_i(c, si);
  return block_sum_f(m, sf);
}

__device__ __forceinline__ int count_ge(const float* p, int n, unsigned b, int* si) {
  int c = 0;
  for (int v = threadIdx.x; v < n; v += kThreads) {
    const float x = p[v];
    if (x >= 0.f && __float_as_uint(x) >= b) ++c;
  }
  return block_sum_i(c, si);
}

__device__ __forceinline__ int count_eq(const float* p, int n, unsigned xb, int* si) {
  int c = 0;
  for (int v = threadIdx.x; v < n; v += kThreads) {
    const float x = p[v];
    if (x >= 0.f && __float_as_uint(x) == xb) ++c;
  }
  return block_sum_i(c, si);
}

// Mass of {key >= b} within the prefix (xb, c).
__device__ __forceinline__ float mass_ge_within(const float* p, int n, unsigned b, unsigned xb, int c, float* sf) {
  float m = 0.f;
  for (int v = threadIdx.x; v < n; v += kThreads) {
    const float x = p[v];
    if (x >= 0.f) {
      const unsigned k = __float_as_uint(x);
      if (k >= b && k > xb) m += x;
    }
  }
  m = block_sum_f(m, sf);
  if (b <= xb) m += (float)c * __uint_as_float(xb);
  return m;
}

// Index of the (r+1)-th token (by index) whose key equals xb; -1 if there are fewer.
__device__ __forceinline__ int nth_equal(const float* p, int n, unsigned xb, int r, int* si, int* result) {
  const int chunk = (n + kThreads - 1) / kThreads;
  const int lo = min(n, (int)threadIdx.x * chunk), hi = min(n, lo + chunk);
  int mine = 0;
  for (int v = lo; v < hi; ++v) {
    const float x = p[v];
    if (x >= 0.f && __float_as_uint(x) == xb) ++mine;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = mine;  // inclusive scan over the warp
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();
  if (threadIdx.x == 0) *result = -1;
  if (lane == 31) si[warp] = inc;
  __syncthreads();
  int before = inc - mine;
  for (int w2 = 0; w2 < warp; ++w2) before += si[w2];
  if (r >= before && r < before + mine) {
    int seen = before;
    for (int v = lo; v < hi; ++v) {
      const float x = p[v];
      if (x >= 0.f && __float_as_uint(x) == xb) {
        if (seen == r) {
          *result = v;
          break;
        }
        ++seen;
      }
    }
  }
  __syncthreads();
  const int out = *result;
  __syncthreads();
  return out;
}

// seeds and offsets are read as pairs of 32-bit words (low word first).
__global__ void __launch_bounds__(kThreads)
    sample_kernel(const float* __restrict__ logits, long long stride, int vocab, const float* __restrict__ temperature,
                  const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
                  const unsigned* __restrict__ seeds, const unsigned* __restrict__ offsets, float* workspace,
                  int* __restrict__ ids) {
  __shared__ float sf[32];
  __shared__ int si[32];
  __shared__ int s_result;
  const int r = blockIdx.x;
  const float* z = logits + (size_t)r * stride;
  float* p = workspace + (size_t)r * vocab;
  const float temp = temperature[r];

  const int imax = block_argmax(z, vocab, true, sf, si);
  const float zmax = sf[0];
  if (temp <= 0.f || imax < 0) {
    if (threadIdx.x == 0) ids[r] = imax;
    return;
  }

  // probabilities; removed tokens are marked -1
  float part = 0.f;
  int allowed = 0;
  for (int v = threadIdx.x; v < vocab; v += kThreads) {
    const float x = z[v];
    float e = -1.f;
    if (x == x && x != -INFINITY) {
      e = expf((x - zmax) / temp);
      part += e;
      ++allowed;
    }
    p[v] = e;
  }
  const float total = block_sum_f(part, sf);
  allowed = block_sum_i(allowed, si);
  for (int v = threadIdx.x; v < vocab; v += kThreads) {
    const float e = p[v];
    if (e >= 0.f) p[v] = e / total;
  }
  __syncthreads();
  const float pmax = 1.0f / total;  // exp(0) / total

  // the whole allowed set as a prefix: every key above 0, and all tokens whose probability underflowed to 0
  unsigned keep_xb = 0u;
  int keep_c = count_eq(p, vocab, 0u, si);
  constexpr int kTopBit = 29;  // probabilities are at most 1 = 0x3F800000, so bits 31 and 30 of a key are 0

  // top-k: the k-th largest key is the largest b with count(key >= b) >= k
  const int k = top_k[r];
  if (k > 0 && k < allowed) {
    unsigned b = 0u;
    for (int bit = kTopBit; bit >= 0; --bit) {
      const unsigned trial = b | (1u << bit);
      if (count_ge(p, vocab, trial, si) >= k) b = trial;
    }
    int above;
    mass_gt(p, vocab, b, above, sf, si);
    keep_xb = b;
    keep_c = k - above;
  }

  // top-p: the crossing token's key is the largest b with (kept mass of keys >= b) >= top_p * kept mass
  const float tp = top_p[r];
  if (tp < 1.0f) {
    const float kept_total = mass_ge_within(p, vocab, 0u, keep_xb, keep_c, sf);
    const float bar = tp * kept_total;
    unsigned b = 0u;
    for (int bit = kTopBit; bit >= 0; --bit) {
      const unsigned trial = b | (1u << bit);
      if (mass_ge_within(p, vocab, trial, keep_xb, keep_c, sf) >= bar) b = trial;
    }
    if (b < keep_xb) b = keep_xb;
    int gt_count;
    const float gt_mass = mass_gt(p, vocab, b, gt_count, sf, si);
    const float x = __uint_as_float(b);
    const int ties = (b == keep_xb) ? keep_c : count_eq(p, vocab, b, si);
    int need = 1;
    if (x > 0.f) {
      need = (int)ceilf((bar - gt_mass) / x);
      if (need < 1) need = 1;
    }
    if (need > ties) need = ties;
    keep_xb = b;
    keep_c = need;
  }

  // min-p: drop p < min_p * p_max; what stays is {key > bits(floor) - 1} when the prefix reached below the floor
  const float mp = min_p[r];
  if (mp > 0.f) {
    const float floor_p = mp * pmax;
    if (__uint_as_float(keep_xb) < floor_p) {
      keep_xb = __float_as_uint(floor_p) - 1u;
      keep_c = 0;
    }
  }

  // the draw: the chosen token's key is the largest b with (kept mass of keys >= b) > u * kept mass
  int above;
  mass_gt(p, vocab, keep_xb, above, sf, si);
  int chosen = -1;
  if (above == 0 && keep_c == 0) {
    chosen = imax;  // min-p above 1 left nothing: the reference keeps the first token of the order
  } else {
    const float mass = mass_ge_within(p, vocab, 0u, keep_xb, keep_c, sf);
    const unsigned r0 = philox4x32_10(offsets[2 * r], offsets[2 * r + 1], 0u, 0u, seeds[2 * r], seeds[2 * r + 1]);
    const float u = (float)(r0 >> 8) * (1.0f / 16777216.0f);
    const float target = u * mass;
    if (mass > target) {
      unsigned b = 0u;
      for (int bit = kTopBit; bit >= 0; --bit) {
        const unsigned trial = b | (1u << bit);
        if (mass_ge_within(p, vocab, trial, keep_xb, keep_c, sf) > target) b = trial;
      }
      if (b < keep_xb) b = keep_xb;
      int gt_count;
      const float gt_mass = mass_gt(p, vocab, b, gt_count, sf, si);
      const float x = __uint_as_float(b);
      const int ties = (b == keep_xb) ? keep_c : count_eq(p, vocab, b, si);
      if (ties > 0) {
        int rnk = 0;
        if (x > 0.f) {
          rnk = (int)floorf((target - gt_mass) / x);
          if (rnk < 0) rnk = 0;
        }
        if (rnk > ties - 1) rnk = ties - 1;
        chosen = nth_equal(p, vocab, b, rnk, si, &s_result);
      }
    }
    if (chosen < 0) {
      // rounding left none: the last kept token, i.e. the smallest kept key and its last kept tie
      unsigned b = keep_xb;
      int ties = keep_c;
      if (ties == 0) {
        b = 0u;  // the smallest key above keep_xb is the largest b with count(key >= b) >= above
        for (int bit = kTopBit; bit >= 0; --bit) {
          const unsigned trial = b | (1u << bit);
          if (count_ge(p, vocab, trial, si) >= above) b = trial;
        }
        ties = count_eq(p, vocab, b, si);
      }
      chosen = ties > 0 ? nth_equal(p, vocab, b, ties - 1, si, &s_result) : imax;
    }
  }
  if (threadIdx.x == 0) ids[r] = chosen;
}

}  // namespace roost

using namespace roost;

extern "C" int roost_argmax_split(const float* logits, int64_t stride, int rows, int vocab, int32_t* ids, int splits, float* part_v,
                                  int32_t* part_i, uint32_t* counters, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && vocab > 0 && stride >= vocab, "argmax: rows, vocab and stride must be consistent");
  ROOST_REQUIRE(splits >= 1 && splits <= 32, "argmax: between 1 and 32 spans a row");
  ROOST_REQUIRE(part_v && part_i && counters, "argmax: the workspace of the spans is missing");
  if (rows == 0) return ROOST_OK;
  if (rows > 65535 * 32) return fail(ROOST_ERR_UNSUPPORTED, "argmax: too many rows");
  argmax_split_kernel<<<dim3(rows, splits), kThreads, 0, (cudaStream_t)stream>>>(logits, (long long)stride, vocab, ids, part_v, part_i, counters);
  return check_launch("argmax");
}

extern "C" int roost_argmax(const float* logits, int64_t stride, int rows, int vocab, int32_t* ids, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && vocab > 0 && stride >= vocab, "argmax: rows, vocab and stride must be consistent");
  if (rows == 0) return ROOST_OK;
  argmax_kernel<<<rows, kThreads, 0, (cudaStream_t)stream>>>(logits, (long long)stride, vocab, ids);
  return check_launch("argmax");
}

extern "C" int roost_sample(const float* logits, int64_t stride, int rows, int vocab, const float* temperature,
                            const int32_t* top_k, const float* top_p, const float* min_p, const uint64_t* seeds,
                            const uint64_t* offsets, float* workspace, int32_t* ids, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && vocab > 0 && stride >= vocab, "sample: rows, vocab and stride must be consistent");
  ROOST_REQUIRE(temperature && top_k && top_p && min_p && seeds && offsets && workspace && ids, "sample: a parameter table is null");
  if (rows == 0) return ROOST_OK;
  ROOST_REQUIRE(((uintptr_t)logits & 3) == 0 && ((uintptr_t)workspace & 3) == 0 && ((uintptr_t)seeds & 3) == 0 &&
                    ((uintptr_t)offsets & 3) == 0,
                "sample: a table is not aligned to its element size");
  sample_kernel<<<rows, kThreads, 0, (cudaStream_t)stream>>>(logits, (long long)stride, vocab, temperature, top_k, top_p, min_p,
                                                            (const unsigned*)seeds, (const unsigned*)offsets, workspace, ids);
  return check_launch("sample");
}
