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
// search for x over the bit patterns of the weights (non-negative floats order like their bits): three passes
// over the row, one per digit of the key, each a histogram of integer masses and a suffix sum (search_key
// below), and a count of ties. Integer sums do not depend on their order, so a row gives the same token in
// any batch and on any run. The masses are rounded to 2^-40 of the largest weight where the reference sums
// doubles over a sorted array: a draw within rounding of an interval's edge may fall to the neighbouring token.
#include <cooperative_groups.h>

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
// Keys are the bit patterns of the weights e = exp((z - max) / T), which order like the probabilities e / total;
// removed tokens hold -1 and are skipped. A weight's mass is the integer round(e * 2^40): integer sums do not depend on
// the order of their terms, so every mass below is exact, the same in any batch and on any run, and histograms may be
// filled with atomic adds. (A weight below 2^-41 has mass 0: all of them together are less than 2^-23 of the largest.)
// a key's 30 significant bits, searched digit by digit, high to low: 11, 11 and 8 bits
__device__ __forceinline__ constexpr int digit_bits(int level) { return level == 2 ? 8 : 11; }
__device__ __forceinline__ constexpr int digit_shift(int level) { return level == 0 ? 19 : (level == 1 ? 8 : 0); }
constexpr int kBuckets = 2048;

struct SearchScratch {
  unsigned long long mass[kBuckets];
  unsigned cnt[kBuckets];
  unsigned long long warp_mass[32];
  unsigned warp_cnt[32];
  unsigned long long found_above_mass;
  unsigned found_above_cnt, found_digit;
  unsigned long long found_mass;   // of the digit itself
  unsigned found_cnt;
};

__device__ __forceinline__ unsigned long long weight_mass(float e) { return __float2ull_rn(e * 1099511627776.0f); }

// The largest key b such that the measure of {keys >= b} within the prefix (xb, c) reaches `target` (is at least it, or
// with `strict` exceeds it); the measure is the mass, or with `by_count` the number of tokens. Three passes over the row,
// one per digit: a histogram of the measure over the digit among the tokens that share the digits chosen so far, a
// suffix sum over the buckets, and the bucket where the sum crosses the target. Leaves in `above_mass` / `above_cnt`
// the mass and count of {keys > b} within the prefix and in `ties` the number of tokens whose key is b (of which the
// prefix holds c when b == xb). Requires that the whole prefix reaches the target.
__device__ unsigned search_key(const float* __restrict__ p, int n, unsigned xb, int c, unsigned long long target, bool strict, bool by_count,
                               SearchScratch& h, unsigned long long& above_mass, unsigned& above_cnt, unsigned& ties) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned prefix = 0u;                 // the digits chosen so far, in place
  unsigned prefix_mask = 0u;
  unsigned long long acc_mass = 0ull;   // measure of the keys above every bucket chosen so far
  unsigned acc_cnt = 0u;
  const unsigned long long xb_mass = weight_mass(__uint_as_float(xb));
  for (int level = 0; level < 3; ++level) {
    const int shift = digit_shift(level), buckets = 1 << digit_bits(level);
    for (int i = threadIdx.x; i < buckets; i += kThreads) {
      h.mass[i] = 0ull;
      h.cnt[i] = 0u;
    }
    __syncthreads();
    constexpr int kAhead = 8;   // loads in flight a thread: the pass is bound by their latency, not by their bytes
    for (int base = 0; base < n; base += kThreads * kAhead) {   // whole warps go round together: the exchange below names all lanes
      float xs[kAhead];
#pragma unroll
      for (int j = 0; j < kAhead; ++j) {
        const int v = base + j * kThreads + (int)threadIdx.x;
        xs[j] = v < n ? p[v] : -1.f;
      }
#pragma unroll
      for (int j = 0; j < kAhead; ++j) {
        const float x = xs[j];
        unsigned digit = 0xffffffffu;   // no token of this search
        unsigned long long w = 0ull;
        if (x >= 0.f) {
          const unsigned k = __float_as_uint(x);
          if ((k & prefix_mask) == prefix && k > xb) {   // the tokens at xb are counted below, c of them
            digit = (k >> shift) & (unsigned)(buckets - 1);
            w = weight_mass(x);
          }
        }
        // a row whose tokens crowd into one bucket (equal logits) would queue a hundred thousand adds on one address:
        // a warp whose lanes all name the same bucket adds once
        if (__match_any_sync(0xffffffffu, digit) == 0xffffffffu) {
          if (digit != 0xffffffffu) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
            if (lane == 0) {
              atomicAdd(&h.mass[digit], w);
              atomicAdd(&h.cnt[digit], 32u);
            }
          }
        } else if (digit != 0xffffffffu) {
          atomicAdd(&h.mass[digit], w);
          atomicAdd(&h.cnt[digit], 1u);
        }
      }
    }
    if (threadIdx.x == 0 && c > 0 && (xb & prefix_mask) == prefix) {
      const unsigned digit = (xb >> shift) & (unsigned)(buckets - 1);
      atomicAdd(&h.mass[digit], xb_mass * (unsigned long long)c);
      atomicAdd(&h.cnt[digit], (unsigned)c);
    }
    __syncthreads();
    // suffix sums, high digits first: thread t holds buckets [per t, per (t + 1)) counted from the top
    const int per = (buckets + kThreads - 1) / kThreads;
    unsigned long long my_mass = 0ull;
    unsigned my_cnt = 0u;
    for (int i = 0; i < per; ++i) {
      const int bkt = buckets - 1 - ((int)threadIdx.x * per + i);
      if (bkt >= 0) {
        my_mass += h.mass[bkt];
        my_cnt += h.cnt[bkt];
      }
    }
    unsigned long long inc_mass = my_mass;   // inclusive scan over the warp, then over the warps
    unsigned inc_cnt = my_cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long tm = __shfl_up_sync(0xffffffffu, inc_mass, o);
      const unsigned tc = __shfl_up_sync(0xffffffffu, inc_cnt, o);
      if (lane >= o) {
        inc_mass += tm;
        inc_cnt += tc;
      }
    }
    if (lane == 31) {
      h.warp_mass[warp] = inc_mass;
      h.warp_cnt[warp] = inc_cnt;
    }
    __syncthreads();
    unsigned long long before_mass = acc_mass + inc_mass - my_mass;
    unsigned before_cnt = acc_cnt + inc_cnt - my_cnt;
    for (int w2 = 0; w2 < warp; ++w2) {
      before_mass += h.warp_mass[w2];
      before_cnt += h.warp_cnt[w2];
    }
    // the bucket where the running measure (from the top) first reaches the target
    for (int i = 0; i < per; ++i) {
      const int bkt = buckets - 1 - ((int)threadIdx.x * per + i);
      if (bkt < 0) break;
      const unsigned long long bm = h.mass[bkt];
      const unsigned bc = h.cnt[bkt];
      const unsigned long long before = by_count ? (unsigned long long)before_cnt : before_mass;
      const unsigned long long with = before + (by_count ? (unsigned long long)bc : bm);
      const bool was = strict ? before > target : before >= target;
      const bool is = strict ? with > target : with >= target;
      if (!was && is) {
        h.found_digit = (unsigned)bkt;
        h.found_above_mass = before_mass;
        h.found_above_cnt = before_cnt;
        h.found_mass = bm;
        h.found_cnt = bc;
      }
      before_mass += bm;
      before_cnt += bc;
    }
    __syncthreads();
    prefix |= h.found_digit << shift;
    prefix_mask |= (unsigned)(buckets - 1) << shift;
    acc_mass = h.found_above_mass;
    acc_cnt = h.found_above_cnt;
    ties = h.found_cnt;
    __syncthreads();
  }
  above_mass = acc_mass;
  above_cnt = acc_cnt;
  return prefix;
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
  __shared__ SearchScratch h;
  __shared__ unsigned long long s_total;
  __shared__ unsigned s_allowed, s_zero;
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

  // the weights e = exp((z - max) / T), at most 1; removed tokens are marked -1
  if (threadIdx.x == 0) {
    s_total = 0ull;
    s_allowed = 0u;
    s_zero = 0u;
  }
  __syncthreads();
  unsigned long long part = 0ull;
  unsigned allowed_mine = 0u, zero_mine = 0u;
  for (int v = threadIdx.x; v < vocab; v += kThreads) {
    const float x = z[v];
    float e = -1.f;
    if (x == x && x != -INFINITY) {
      e = expf((x - zmax) / temp);
      part += weight_mass(e);
      ++allowed_mine;
      zero_mine += e == 0.f ? 1u : 0u;
    }
    p[v] = e;
  }
  atomicAdd(&s_total, part);
  atomicAdd(&s_allowed, allowed_mine);
  atomicAdd(&s_zero, zero_mine);
  __syncthreads();
  const int allowed = (int)s_allowed;

  // the whole allowed set as a prefix: every key above 0, and all tokens whose weight underflowed to 0
  unsigned keep_xb = 0u;
  int keep_c = (int)s_zero;
  unsigned long long kept_mass = s_total;   // mass of the prefix (keep_xb, keep_c)
  unsigned long long above_mass;
  unsigned above_cnt, ties;

  // top-k: the k-th largest key is the largest b with count(key >= b) >= k
  const int k = top_k[r];
  if (k > 0 && k < allowed) {
    const unsigned b = search_key(p, vocab, keep_xb, keep_c, (unsigned long long)k, false, true, h, above_mass, above_cnt, ties);
    keep_xb = b;
    keep_c = k - (int)above_cnt;
    kept_mass = above_mass + (unsigned long long)keep_c * weight_mass(__uint_as_float(b));
  }

  // top-p: the crossing token's key is the largest b with (kept mass of keys >= b) >= top_p * kept mass
  const float tp = top_p[r];
  if (tp < 1.0f && kept_mass > 0ull) {
    unsigned long long bar = (unsigned long long)ceil((double)tp * (double)kept_mass);
    if (bar > kept_mass) bar = kept_mass;
    if (bar < 1ull) bar = 1ull;
    const unsigned b = search_key(p, vocab, keep_xb, keep_c, bar, false, false, h, above_mass, above_cnt, ties);
    const unsigned long long x = weight_mass(__uint_as_float(b));
    const int have = (b == keep_xb) ? keep_c : (int)ties;
    int need = 1;
    if (x > 0ull && bar > above_mass) {
      const unsigned long long q = (bar - above_mass + x - 1ull) / x;
      need = q > (unsigned long long)have ? have : (int)q;
      if (need < 1) need = 1;
    }
    if (need > have) need = have;
    keep_xb = b;
    keep_c = need;
    kept_mass = above_mass + (unsigned long long)need * x;
  }

  // min-p: drop e < min_p (the largest weight is 1); what stays is {key > bits(min_p) - 1} when the prefix reached below
  const float mp = min_p[r];
  bool recount = false;
  if (mp > 0.f && __uint_as_float(keep_xb) < mp) {
    keep_xb = __float_as_uint(mp) - 1u;
    keep_c = 0;
    recount = true;
  }

  // the draw: the chosen token's key is the largest b with (kept mass of keys >= b) > u * kept mass
  int chosen = -1;
  if (recount) {
    // the mass above the new floor: one pass
    unsigned long long m = 0ull;
    for (int v = threadIdx.x; v < vocab; v += kThreads) {
      const float x = p[v];
      if (x >= 0.f && __float_as_uint(x) > keep_xb) m += weight_mass(x);
    }
    __syncthreads();
    if (threadIdx.x == 0) s_total = 0ull;
    __syncthreads();
    atomicAdd(&s_total, m);
    __syncthreads();
    kept_mass = s_total;
  }
  if (kept_mass == 0ull) {
    chosen = imax;  // min-p above 1 left nothing (or every kept weight's mass is 0): the reference keeps the first token of the order
  } else {
    const unsigned r0 = philox4x32_10(offsets[2 * r], offsets[2 * r + 1], 0u, 0u, seeds[2 * r], seeds[2 * r + 1]);
    const double u = (double)(r0 >> 8) * (1.0 / 16777216.0);
    unsigned long long target = (unsigned long long)(u * (double)kept_mass);   // below kept_mass, since u < 1
    if (target >= kept_mass) target = kept_mass - 1ull;
    const unsigned b = search_key(p, vocab, keep_xb, keep_c, target, true, false, h, above_mass, above_cnt, ties);
    const unsigned long long x = weight_mass(__uint_as_float(b));
    const int have = (b == keep_xb) ? keep_c : (int)ties;
    int rnk = 0;
    if (x > 0ull && target >= above_mass) {
      const unsigned long long q = (target - above_mass) / x;   // tokens of this key wholly at or below the target
      rnk = q > (unsigned long long)(have - 1) ? have - 1 : (int)q;
    }
    if (have > 0) chosen = nth_equal(p, vocab, b, rnk, si, &s_result);
    if (chosen < 0) chosen = imax;
  }
  if (threadIdx.x == 0) ids[r] = chosen;
}

// ------------------------------------------------------------------------------------------------ a row on a cluster of CTAs
// One SM reads a row of a large vocabulary at about 30 GB/s, and a search makes several passes over it: a block a row
// takes 460 us at 151,936 tokens. Here a cluster of eight (or four) CTAs takes a row: each keeps its part of the row's
// weights in shared memory, so every pass after the first reads shared memory, and the CTAs combine what they find through
// each other's shared memory: histograms are reduced bucket range by bucket range (CTA c owns its share of the buckets),
// the range that holds the crossing is found from the ranges' totals, and its owner finds the bucket and tells the
// others. Every sum is an integer sum, so the result is the single block's, bit for bit.
namespace cg = cooperative_groups;
// Eight CTAs a row while at most eight rows are sampled (fifteen or so clusters of eight run at once); four from there on
// (37 of them at once, one CTA an SM with its quarter of the row in shared memory), so that 64 rows take two rounds, not five.
constexpr int kClusterMaxCtas = 8, kClusterMinCtas = 4;
constexpr int kSliceFloats8 = 24576;   // of a row, in a CTA's shared memory (96 KB): rows of up to 196,608 tokens
constexpr int kSliceFloats4 = 40960;   // 160 KB: rows of up to 163,840 tokens

struct ClusterScratch {
  SearchScratch h;                                   // this CTA's histogram of its slice
  unsigned long long own_mass[kBuckets / kClusterMinCtas];   // the cluster's totals of the buckets this CTA owns
  unsigned own_cnt[kBuckets / kClusterMinCtas];
  unsigned long long own_total_mass;
  unsigned own_total_cnt;
  unsigned long long pub_u64[2][2];                  // all-reduce slots, used in turn
  unsigned pub_u32[2][2];
  float am_val;                                      // this CTA's best logit and its index
  int am_idx;
  unsigned long long found_above_mass, found_mass;   // what the owner of the crossing bucket tells the others
  unsigned found_above_cnt, found_cnt, found_digit;
  int crossing_rank;
  unsigned long long crossing_above_mass;
  unsigned crossing_above_cnt;
  unsigned ties_local;
};

__device__ __forceinline__ unsigned long long warp_sum_u64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sums (a, b) over the cluster; every thread of every CTA calls it and gets the totals.
__device__ void cluster_sum2(cg::cluster_group& cluster, ClusterScratch& cs, int& turn, unsigned long long& a, unsigned& b) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  a = warp_sum_u64(a);
  b = (unsigned)warp_sum_i((int)b);
  __syncthreads();
  if (lane == 0) {
    cs.h.warp_mass[warp] = a;
    cs.h.warp_cnt[warp] = b;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long ta = 0ull;
    unsigned tb = 0u;
    for (int w = 0; w < kThreads / 32; ++w) {
      ta += cs.h.warp_mass[w];
      tb += cs.h.warp_cnt[w];
    }
    cs.pub_u64[turn][0] = ta;
    cs.pub_u32[turn][0] = tb;
  }
  cluster.sync();
  unsigned long long ta = 0ull;
  unsigned tb = 0u;
  for (int r = 0; r < (int)cluster.num_blocks(); ++r) {
    const ClusterScratch* o = cluster.map_shared_rank(&cs, r);
    ta += o->pub_u64[turn][0];
    tb += o->pub_u32[turn][0];
  }
  a = ta;
  b = tb;
  turn ^= 1;
}

// search_key over the cluster: the same definition and the same result, the row's weights in the CTAs' slices.
__device__ unsigned cluster_search_key(cg::cluster_group& cluster, ClusterScratch& cs, const float* __restrict__ slice, int n_local, unsigned xb,
                                       int c, unsigned long long target, bool strict, bool by_count, unsigned long long& above_mass,
                                       unsigned& above_cnt, unsigned& ties) {
  const int rank = (int)cluster.block_rank(), ctas = (int)cluster.num_blocks();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned prefix = 0u, prefix_mask = 0u;
  unsigned long long acc_mass = 0ull;
  unsigned acc_cnt = 0u;
  const unsigned long long xb_mass = weight_mass(__uint_as_float(xb));
  auto reaches = [&](unsigned long long mass, unsigned cnt) {
    const unsigned long long m = by_count ? (unsigned long long)cnt : mass;
    return strict ? m > target : m >= target;
  };
  for (int level = 0; level < 3; ++level) {
    const int shift = digit_shift(level), buckets = 1 << digit_bits(level), own = buckets / ctas;
    for (int i = threadIdx.x; i < buckets; i += kThreads) {
      cs.h.mass[i] = 0ull;
      cs.h.cnt[i] = 0u;
    }
    __syncthreads();
    for (int v = threadIdx.x; v < n_local; v += kThreads) {
      const float x = slice[v];
      if (x < 0.f) continue;
      const unsigned k = __float_as_uint(x);
      if ((k & prefix_mask) != prefix || k <= xb) continue;   // the tokens at xb are counted below, c of them
      const unsigned digit = (k >> shift) & (unsigned)(buckets - 1);
      atomicAdd(&cs.h.mass[digit], weight_mass(x));
      atomicAdd(&cs.h.cnt[digit], 1u);
    }
    if (rank == 0 && threadIdx.x == 0 && c > 0 && (xb & prefix_mask) == prefix) {
      const unsigned digit = (xb >> shift) & (unsigned)(buckets - 1);
      atomicAdd(&cs.h.mass[digit], xb_mass * (unsigned long long)c);
      atomicAdd(&cs.h.cnt[digit], (unsigned)c);
    }
    cluster.sync();
    // the cluster's totals of the buckets this CTA owns, and their sum
    unsigned long long mine_mass = 0ull;
    unsigned mine_cnt = 0u;
    if ((int)threadIdx.x < own) {
      const int bkt = rank * own + (int)threadIdx.x;
      for (int r = 0; r < ctas; ++r) {
        const ClusterScratch* o = cluster.map_shared_rank(&cs, r);
        mine_mass += o->h.mass[bkt];
        mine_cnt += o->h.cnt[bkt];
      }
      cs.own_mass[threadIdx.x] = mine_mass;
      cs.own_cnt[threadIdx.x] = mine_cnt;
    }
    {
      unsigned long long wm = warp_sum_u64(mine_mass);
      unsigned wc = (unsigned)warp_sum_i((int)mine_cnt);
      if (lane == 0) {
        cs.h.warp_mass[warp] = wm;
        cs.h.warp_cnt[warp] = wc;
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        unsigned long long tm = 0ull;
        unsigned tc = 0u;
        for (int w = 0; w < (own + 31) / 32; ++w) {
          tm += cs.h.warp_mass[w];
          tc += cs.h.warp_cnt[w];
        }
        cs.own_total_mass = tm;
        cs.own_total_cnt = tc;
      }
    }
    cluster.sync();
    // the range of buckets in which the running measure (from the top) first reaches the target: the same in every CTA
    if (threadIdx.x == 0) {
      unsigned long long m = acc_mass;
      unsigned n = acc_cnt;
      int at = 0;
      for (int r = ctas - 1; r >= 0; --r) {
        const ClusterScratch* o = cluster.map_shared_rank(&cs, r);
        const unsigned long long rm = o->own_total_mass;
        const unsigned rc = o->own_total_cnt;
        if (reaches(m + rm, n + rc)) {
          at = r;
          break;
        }
        m += rm;
        n += rc;
      }
      cs.crossing_rank = at;
      cs.crossing_above_mass = m;
      cs.crossing_above_cnt = n;
    }
    __syncthreads();
    const int owner = cs.crossing_rank;
    if (rank == owner) {
      // the bucket within this CTA's range: a scan from the range's top bucket down, one bucket a thread
      const int t = (int)threadIdx.x;
      const bool in = t < own;
      const int bkt = rank * own + (own - 1 - t);
      const unsigned long long bm = in ? cs.own_mass[own - 1 - t] : 0ull;
      const unsigned bc = in ? cs.own_cnt[own - 1 - t] : 0u;
      unsigned long long inc_m = bm;
      unsigned inc_c = bc;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long tm = __shfl_up_sync(0xffffffffu, inc_m, o);
        const unsigned tc = __shfl_up_sync(0xffffffffu, inc_c, o);
        if (lane >= o) {
          inc_m += tm;
          inc_c += tc;
        }
      }
      __syncthreads();
      if (lane == 31) {
        cs.h.warp_mass[warp] = inc_m;
        cs.h.warp_cnt[warp] = inc_c;
      }
      __syncthreads();
      unsigned long long before_m = cs.crossing_above_mass + inc_m - bm;
      unsigned before_c = cs.crossing_above_cnt + inc_c - bc;
      for (int w = 0; w < warp; ++w) {
        before_m += cs.h.warp_mass[w];
        before_c += cs.h.warp_cnt[w];
      }
      if (in && !reaches(before_m, before_c) && reaches(before_m + bm, before_c + bc)) {
        cs.found_digit = (unsigned)bkt;
        cs.found_above_mass = before_m;
        cs.found_above_cnt = before_c;
        cs.found_mass = bm;
        cs.found_cnt = bc;
      }
    }
    cluster.sync();
    const ClusterScratch* o = cluster.map_shared_rank(&cs, owner);
    prefix |= o->found_digit << shift;
    prefix_mask |= (unsigned)(buckets - 1) << shift;
    acc_mass = o->found_above_mass;
    acc_cnt = o->found_above_cnt;
    ties = o->found_cnt;
  }
  cluster.sync();   // the owner's word has been read by everyone before a later search writes it again
  above_mass = acc_mass;
  above_cnt = acc_cnt;
  return prefix;
}

__global__ void __launch_bounds__(kThreads)
    sample_cluster_kernel(const float* __restrict__ logits, long long stride, int vocab, const float* __restrict__ temperature,
                          const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
                          const unsigned* __restrict__ seeds, const unsigned* __restrict__ offsets, int* __restrict__ ids) {
  extern __shared__ float slice[];
  __shared__ float sf[32];
  __shared__ int si[32];
  __shared__ int s_result;
  __shared__ ClusterScratch cs;
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank(), ctas = (int)cluster.num_blocks();
  const int r = blockIdx.x / ctas;
  const int span = (((vocab + ctas - 1) / ctas) + 3) & ~3;
  const int lo = min(vocab, rank * span), n_local = min(vocab, lo + span) - lo;
  const float* z = logits + (size_t)r * stride + lo;
  const float temp = temperature[r];
  int turn = 0;

  // the row's best logit: every CTA's best, combined in rank order
  const int local_best = block_argmax(z, n_local, true, sf, si);
  if (threadIdx.x == 0) {
    cs.am_val = sf[0];
    cs.am_idx = local_best < 0 ? -1 : local_best + lo;
  }
  cluster.sync();
  float zmax = 0.f;
  int imax = -1;
  for (int c = 0; c < ctas; ++c) {
    const ClusterScratch* o = cluster.map_shared_rank(&cs, c);
    const float ov = o->am_val;
    const int oi = o->am_idx;
    if (!better(zmax, imax, ov, oi)) {
      zmax = ov;
      imax = oi;
    }
  }
  if (temp <= 0.f || imax < 0) {
    if (rank == 0 && threadIdx.x == 0) ids[r] = imax;
    cluster.sync();   // nobody leaves while another CTA still reads its shared memory
    return;
  }

  // the weights e = exp((z - max) / T) of this CTA's slice, at most 1; removed tokens are marked -1
  unsigned long long total = 0ull;
  unsigned allowed_u = 0u, zeros_mine = 0u;
  for (int v = threadIdx.x; v < n_local; v += kThreads) {
    const float x = z[v];
    float e = -1.f;
    if (x == x && x != -INFINITY) {
      e = expf((x - zmax) / temp);
      total += weight_mass(e);
      ++allowed_u;
      zeros_mine += e == 0.f ? 1u : 0u;
    }
    slice[v] = e;
  }
  cluster_sum2(cluster, cs, turn, total, allowed_u);
  unsigned long long zeros64 = zeros_mine;
  unsigned dummy = 0u;
  cluster_sum2(cluster, cs, turn, zeros64, dummy);
  const int allowed = (int)allowed_u;

  unsigned keep_xb = 0u;
  int keep_c = (int)zeros64;
  unsigned long long kept_mass = total;
  unsigned long long above_mass;
  unsigned above_cnt, ties;

  const int k = top_k[r];
  if (k > 0 && k < allowed) {
    const unsigned b = cluster_search_key(cluster, cs, slice, n_local, keep_xb, keep_c, (unsigned long long)k, false, true, above_mass, above_cnt, ties);
    keep_xb = b;
    keep_c = k - (int)above_cnt;
    kept_mass = above_mass + (unsigned long long)keep_c * weight_mass(__uint_as_float(b));
  }

  const float tp = top_p[r];
  if (tp < 1.0f && kept_mass > 0ull) {
    unsigned long long bar = (unsigned long long)ceil((double)tp * (double)kept_mass);
    if (bar > kept_mass) bar = kept_mass;
    if (bar < 1ull) bar = 1ull;
    const unsigned b = cluster_search_key(cluster, cs, slice, n_local, keep_xb, keep_c, bar, false, false, above_mass, above_cnt, ties);
    const unsigned long long x = weight_mass(__uint_as_float(b));
    const int have = (b == keep_xb) ? keep_c : (int)ties;
    int need = 1;
    if (x > 0ull && bar > above_mass) {
      const unsigned long long q = (bar - above_mass + x - 1ull) / x;
      need = q > (unsigned long long)have ? have : (int)q;
      if (need < 1) need = 1;
    }
    if (need > have) need = have;
    keep_xb = b;
    keep_c = need;
    kept_mass = above_mass + (unsigned long long)need * x;
  }

  const float mp = min_p[r];
  if (mp > 0.f && __uint_as_float(keep_xb) < mp) {
    keep_xb = __float_as_uint(mp) - 1u;
    keep_c = 0;
    unsigned long long m = 0ull;
    for (int v = threadIdx.x; v < n_local; v += kThreads) {
      const float x = slice[v];
      if (x >= 0.f && __float_as_uint(x) > keep_xb) m += weight_mass(x);
    }
    unsigned none = 0u;
    cluster_sum2(cluster, cs, turn, m, none);
    kept_mass = m;
  }

  int chosen = -1;          // meaningful in the CTA that writes the row's id
  bool mine = rank == 0;    // which CTA that is
  if (kept_mass == 0ull) {
    chosen = imax;
  } else {
    const unsigned r0 = philox4x32_10(offsets[2 * r], offsets[2 * r + 1], 0u, 0u, seeds[2 * r], seeds[2 * r + 1]);
    const double u = (double)(r0 >> 8) * (1.0 / 16777216.0);
    unsigned long long target = (unsigned long long)(u * (double)kept_mass);
    if (target >= kept_mass) target = kept_mass - 1ull;
    const unsigned b = cluster_search_key(cluster, cs, slice, n_local, keep_xb, keep_c, target, true, false, above_mass, above_cnt, ties);
    const unsigned long long x = weight_mass(__uint_as_float(b));
    const int have = (b == keep_xb) ? keep_c : (int)ties;
    int rnk = 0;
    if (x > 0ull && target >= above_mass) {
      const unsigned long long q = (target - above_mass) / x;
      rnk = q > (unsigned long long)(have - 1) ? have - 1 : (int)q;
    }
    // the (rnk + 1)-th token of key b by index: the slices are in index order, so count them slice by slice
    unsigned here = 0u;
    for (int v = threadIdx.x; v < n_local; v += kThreads) {
      const float xv = slice[v];
      here += (xv >= 0.f && __float_as_uint(xv) == b) ? 1u : 0u;
    }
    here = (unsigned)block_sum_i((int)here, si);
    if (threadIdx.x == 0) cs.ties_local = here;
    cluster.sync();
    int before = 0, owner = -1;
    for (int c2 = 0; c2 < ctas; ++c2) {
      const unsigned t = cluster.map_shared_rank(&cs, c2)->ties_local;
      if (owner < 0 && have > 0 && rnk < before + (int)t) owner = c2;
      if (owner < 0) before += (int)t;
    }
    if (owner < 0) {
      chosen = imax;   // no token of that key (cannot be, with exact masses): the row's best
    } else {
      mine = rank == owner;
      if (mine) {
        const int local = nth_equal(slice, n_local, b, rnk - before, si, &s_result);
        chosen = local < 0 ? imax : local + lo;
      }
    }
  }
  if (mine && threadIdx.x == 0) ids[r] = chosen;
  cluster.sync();   // nobody leaves while another CTA still reads its shared memory
}

// ------------------------------------------------------------------------------------------------ penalties and logprobs
// The reference's penalties, in its float32 form (src/Starlings.Roost.Ops/CpuOps.Sampling.cs:195-237: separate divides,
// multiplies and subtracts, in vLLM's order): with c the token's count in the request's output so far and `seen` true when
// c > 0 or the token is in the prompt, a seen logit x becomes x / repetition if it is above 0 and x * repetition otherwise;
// then x - frequency * c; then, when c > 0, x - presence. After the penalties a token whose bit is 0 in the slot's mask
// (bit v % 32 of word v / 32) is removed (-inf), as the reference removes it (:18-19). A row whose slot is negative is
// copied as it is.
__global__ void penalise_kernel(const float* __restrict__ logits, long long stride, int vocab, float* __restrict__ out,
                                const int* __restrict__ counts, const unsigned* __restrict__ prompt_bits, const unsigned* __restrict__ mask_bits,
                                int words, const int* __restrict__ row_slot, const float* __restrict__ repetition,
                                const float* __restrict__ presence, const float* __restrict__ frequency) {
  const int r = blockIdx.y;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= vocab) return;
  float x = logits[(size_t)r * stride + v];
  const int slot = row_slot[r];
  if (slot >= 0) {
    const int c = counts[(size_t)slot * vocab + v];
    const bool seen = c > 0 || ((prompt_bits[(size_t)slot * words + (v >> 5)] >> (v & 31)) & 1u) != 0u;
    if (seen) {
      const float rep = repetition[r];
      x = x > 0.f ? __fdiv_rn(x, rep) : __fmul_rn(x, rep);
    }
    x = __fsub_rn(x, __fmul_rn(frequency[r], (float)c));
    if (c > 0) x = __fsub_rn(x, presence[r]);
    if (mask_bits != nullptr && ((mask_bits[(size_t)slot * words + (v >> 5)] >> (v & 31)) & 1u) == 0u) x = -INFINITY;
  }
  out[(size_t)r * vocab + v] = x;
}

// counts[slot of row r][ids[r]] += 1 for the rows that have a slot and a token
__global__ void count_tokens_kernel(int* __restrict__ counts, int vocab, const int* __restrict__ row_slot, const int* __restrict__ ids, int rows) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int slot = row_slot[r], id = ids[r];
  if (slot >= 0 && id >= 0 && id < vocab) atomicAdd(&counts[(size_t)slot * vocab + id], 1);
}

// the bits of one slot's prompt tokens
__global__ void prompt_bits_kernel(unsigned* __restrict__ bits, const int* __restrict__ ids, int n, int vocab) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int id = ids[i];
  if (id >= 0 && id < vocab) atomicOr(&bits[id >> 5], 1u << (id & 31));
}

// Index of the largest logit that comes after (px, pv) in the order "value descending, index ascending" (NaN never; pv < 0:
// the largest of all); -1 when there is none. The value is left in sf[0].
__device__ __forceinline__ int block_argmax_after(const float* z, int n, float px, int pv, float* sf, int* si) {
  float bv = 0.f;
  int bi = -1;
  for (int v = threadIdx.x; v < n; v += kThreads) {
    const float x = z[v];
    if (x != x) continue;
    if (pv >= 0 && !(x < px || (x == px && v > pv))) continue;
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

// The log-softmax of the raw logits at the chosen token, and the `top` highest raw logits with theirs
// (src/Starlings.Roost.Ops/CpuOps.Sampling.cs:539-603): the maximum over the non-NaN logits, the sum of exp(x - max) over
// them (a thread's strided partial sums, then a tree over the block in a fixed order: the same bits on every run), its
// logarithm, and (x - max) - log(sum) for a token. A row without a chosen token gets -inf; missing top entries are id -1.
__global__ void __launch_bounds__(kThreads) logprob_kernel(const float* __restrict__ logits, long long stride, int vocab,
                                                          const int* __restrict__ ids, float* __restrict__ logprob, int top,
                                                          int* __restrict__ top_ids, float* __restrict__ top_vals) {
  __shared__ float sf[32];
  __shared__ int si[32];
  const int r = blockIdx.x;
  const float* z = logits + (size_t)r * stride;
  const int first = block_argmax_after(z, vocab, 0.f, -1, sf, si);
  const float zmax = sf[0];
  float part = 0.f;
  if (first >= 0) {
    for (int v = threadIdx.x; v < vocab; v += kThreads) {
      const float x = z[v];
      if (x == x) part += expf(x - zmax);
    }
  }
  const float sum = block_sum_f(part, sf);
  const float lse = logf(sum);
  if (threadIdx.x == 0 && logprob != nullptr) {
    const int id = ids[r];
    logprob[r] = (id < 0 || id >= vocab || first < 0) ? -INFINITY : (z[id] - zmax) - lse;
  }
  float px = zmax;
  int pv = first;
  for (int i = 0; i < top; ++i) {   // uniform in the block: pv is the same in every thread
    const int v = i == 0 ? first : (pv < 0 ? -1 : block_argmax_after(z, vocab, px, pv, sf, si));
    if (i > 0 && v >= 0) px = sf[0];
    pv = v;
    if (threadIdx.x == 0) {
      top_ids[(size_t)r * top + i] = v;
      top_vals[(size_t)r * top + i] = v < 0 ? -INFINITY : (z[v] - zmax) - lse;
    }
  }
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
  // a cluster of CTAs a row while a row's eighth fits a CTA's shared memory (and the vocabulary is worth eight CTAs);
  // else a block a row over the workspace
  // measured at 151,936 tokens: 8 rows 115 us and 16 rows 204 us with clusters of eight; 17 and 32 rows 137 us, 64 rows
  // 255 us with clusters of four (450 us with eight)
  const int ctas = rows <= 8 ? kClusterMaxCtas : kClusterMinCtas;
  const int slice_cap = ctas == kClusterMaxCtas ? kSliceFloats8 : kSliceFloats4;
  if (vocab >= 4096 && vocab <= ctas * slice_cap && rows <= 65535 / ctas * ctas) {
    const int span = (((vocab + ctas - 1) / ctas) + 3) & ~3;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
      cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(kSliceFloats4 * sizeof(float)));
      attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows * ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = (size_t)span * sizeof(float);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)ctas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, sample_cluster_kernel, logits, (long long)stride, vocab, temperature, top_k, top_p, min_p, (const unsigned*)seeds,
                       (const unsigned*)offsets, ids);
    return check_launch("sample (cluster)");
  }
  sample_kernel<<<rows, kThreads, 0, (cudaStream_t)stream>>>(logits, (long long)stride, vocab, temperature, top_k, top_p, min_p,
                                                            (const unsigned*)seeds, (const unsigned*)offsets, workspace, ids);
  return check_launch("sample");
}

extern "C" int roost_sample_penalise(const float* logits, int64_t stride, int rows, int vocab, float* out, const int32_t* counts,
                                     const uint32_t* prompt_bits, const uint32_t* mask_bits, const int32_t* row_slot, const float* repetition,
                                     const float* presence, const float* frequency, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && vocab > 0 && stride >= vocab, "sample_penalise: rows, vocab and stride must be consistent");
  ROOST_REQUIRE(logits && out && counts && prompt_bits && row_slot && repetition && presence && frequency, "sample_penalise: a table is null");
  if (rows == 0) return ROOST_OK;
  if (rows > 65535) return fail(ROOST_ERR_UNSUPPORTED, "sample_penalise: more than 65535 rows");
  penalise_kernel<<<dim3((vocab + 255) / 256, rows), 256, 0, (cudaStream_t)stream>>>(logits, (long long)stride, vocab, out, counts, prompt_bits,
                                                                                    mask_bits, (vocab + 31) / 32, row_slot, repetition, presence,
                                                                                    frequency);
  return check_launch("sample_penalise");
}

extern "C" int roost_sample_count_tokens(int32_t* counts, int vocab, const int32_t* row_slot, const int32_t* ids, int rows, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && vocab > 0 && counts && row_slot && ids, "sample_count_tokens: a table is null or a size is not positive");
  if (rows == 0) return ROOST_OK;
  count_tokens_kernel<<<(rows + 127) / 128, 128, 0, (cudaStream_t)stream>>>(counts, vocab, row_slot, ids, rows);
  return check_launch("sample_count_tokens");
}

extern "C" int roost_sample_prompt_bits(uint32_t* bits, const int32_t* ids, int n, int vocab, roost_stream_t stream) {
  ROOST_REQUIRE(n >= 0 && vocab > 0 && bits && (ids || n == 0), "sample_prompt_bits: a table is null or a size is not positive");
  if (n == 0) return ROOST_OK;
  prompt_bits_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(bits, ids, n, vocab);
  return check_launch("sample_prompt_bits");
}

extern "C" int roost_sample_logprobs(const float* logits, int64_t stride, int rows, int vocab, const int32_t* ids, float* logprob, int top,
                                     int32_t* top_ids, float* top_vals, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && vocab > 0 && stride >= vocab, "sample_logprobs: rows, vocab and stride must be consistent");
  ROOST_REQUIRE(top >= 0 && top <= vocab, "sample_logprobs: top is outside [0, vocab]");
  ROOST_REQUIRE(logits && (logprob == nullptr || ids) && (top == 0 || (top_ids && top_vals)), "sample_logprobs: a table is null");
  if (rows == 0) return ROOST_OK;
  logprob_kernel<<<rows, kThreads, 0, (cudaStream_t)stream>>>(logits, (long long)stride, vocab, ids, logprob, top, top_ids, top_vals);
  return check_launch("sample_logprobs");
}
