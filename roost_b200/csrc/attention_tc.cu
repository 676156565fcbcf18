// Causal grouped-query attention over the paged cache for prompt portions (rows with more than 16 packed rows), on the
// fifth-generation tensor cores: both products are tcgen05.mma with the accumulators in tensor memory, and the softmax
// weights go from registers to tensor memory, where the second product reads them as its first operand.
//
// Definition and numerics as in attention_mma.cu (src/Starlings.Roost.Ops/CpuOps.cs:181-298; 32-bit scores, maxima,
// exponentials, sums and output accumulation; the softmax weights rounded to bfloat16 as the operand of the second
// product, kernels/README.md:234-236). A CTA owns one or two groups of 128 packed rows (token r / G, head r % G) of one
// request and one key/value head and walks the keys in tiles of 128 at fixed absolute positions, so a row's bits do not
// depend on how the prompt was cut or on what else is in the batch.
//   warp 0 (producer): one 5-D tensor copy per row group brings its Q tile [128 rows x D] into 128-byte-swizzled shared
//     memory; per key tile it looks the pages up and its lanes issue the copies side by side: per page one copy per
//     64-column block of the keys, placed so that the tile's 128 key rows are consecutive in each block (one product then
//     takes them all), and one copy of the values. Keys and values have rings of their own: a tile's keys are free again
//     as soon as its scores are computed, its values only after the second product a tile later.
//   warp 1 (issuer, one lane): per key tile and row group, O += P V of the tile before (one product per 16 keys:
//     M 128, N = D, K 16, with P in tensor memory and V as the N-major operand exactly as the copy left it) and
//     S = Q K^T of this tile (M 128, N 128, K = D) into score columns of the group. With two row groups each has one set
//     of score columns and the products of one group run while the other group's softmax does; a CTA with one row group
//     has two sets and computes the scores of a tile while the softmax of the tile before runs.
//   warps 2.. (softmax, one thread a row, four warps a row group): read the row's 128 scores from tensor memory, scale,
//     mask by position, keep the running maximum and sum, write the weights as bfloat16 pairs over the scores they came
//     from, and at the end divide the accumulator by the sum and write the row out. The maximum a row's weights are taken
//     against moves only when the new maximum exceeds it by more than 2^8 (the weights then stay below 2^8, well inside
//     bfloat16's and float32's range, and the quotient at the end is the same): the row of the output accumulator is
//     rescaled in tensor memory only then.
// Value rows at positions the request does not hold yet (the rest of its last page) or before the CTA's first visible key
// are zeroed in shared memory before the second product, so that whatever the pool holds there cannot reach a result;
// their scores are masked by position. Every wait is bounded (see tma.cuh): a wait given up raises the CTA's abort flag
// and records a code that roost_attention_status() returns.
#include "tcgen05.cuh"

namespace roost {

constexpr float kLog2eTc = 1.4426950408889634f;
constexpr int kTcRows = 128;   // packed rows of a row group
constexpr int kTcKeys = 128;   // keys of a tile
constexpr float kTcLazyRescale = 8.0f;   // a row's reference maximum moves when the new one exceeds it by more than this (log2 units)
__device__ int g_attention_tc_error = 0;

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3, int c4) {
  asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];\n" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
               : "memory");
}

// 2^x in one special-function instruction (inputs here are at most 8 or -inf; results below 2^-126 flush to zero)
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

template <int D, int NG>
struct TcCfg {
  // what fits beside NG Q tiles in 227 KB: a key tile and a value tile are 128 x D x 2 bytes each
  static constexpr int kKStages = D == 128 ? (NG == 1 ? 3 : 2) : 3;
  static constexpr int kVStages = D == 128 ? 2 : 3;
  static constexpr uint32_t kTile = kTcKeys * D * 2;
  static constexpr size_t kSmem = (size_t)NG * kTcRows * D * 2 + (size_t)(kKStages + kVStages) * kTile + 1024;
};

// work[i] = (batch row, first packed row of the item's NG x 128 rows); an item is run once for every key/value head.
// The grid is persistent: CTA c takes the (item, head) pairs c, c + gridDim.x, ... of the list, which the host has sorted
// longest first. Tensor memory and the barriers are set up once; the rings of keys and values, the score columns and the
// barriers' phases run on from one pair to the next, so the copies of the next pair start while the last tiles of this
// one are still being computed.
template <int D, int RPC, int NG>
__global__ void __launch_bounds__(64 + NG * 128, 1)
    attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ q_indptr,
                                const int32_t* __restrict__ kv_lens, const int32_t* __restrict__ kv_indptr,
                                const int32_t* __restrict__ kv_indices, const int2* __restrict__ work, int items, int q_heads, int kv_heads,
                                int page_size, float scale_log2, int window) {
  using Cfg = TcCfg<D, NG>;
  constexpr int BM = kTcRows, TK = kTcKeys, KS = Cfg::kKStages, VS = Cfg::kVStages, NP = TK / RPC, CB = D / 64;
  constexpr uint32_t kQBytes = BM * D * 2;                  // one row group's Q tile
  constexpr uint32_t kTile = Cfg::kTile;                    // keys, or values, of TK positions
  constexpr uint32_t kVPage = CB * RPC * 128;               // the values page copy by page copy: [column block][RPC rows][128 B]
  constexpr int kOps = NP * (CB + 1);                       // copies a tile takes: per page one per column block of keys, one of values
  static_assert(kOps <= 32, "one lane a copy");
  constexpr int SB = NG == 1 ? 2 : 1;                       // sets of score columns a row group has
  constexpr uint32_t kGroupCols = SB * TK + D;              // tensor-memory columns of a row group: the scores (the weights over them) and the output
  constexpr uint32_t kTmemCols = NG * kGroupCols <= 256 ? 256 : 512;
  static_assert(NG * kGroupCols <= 512, "tensor memory has 512 columns");
  constexpr int kGroupBars = 2 * SB + 1;                    // s_full[SB], p_full[SB], o_done
  constexpr int kGroupThreads = 128;                        // one thread a row
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = ((uint32_t)__cvta_generic_to_shared(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;
  const uint32_t k_smem = q_smem + NG * kQBytes;
  const uint32_t v_smem = k_smem + KS * kTile;
  __shared__ __align__(8) uint64_t bars[2 + 2 * KS + 2 * VS + NG * kGroupBars];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(bars);
  const uint32_t q_full = bar0, q_empty = bar0 + 8u;
  auto k_full = [&](int s) { return bar0 + 8u * (2 + s); };
  auto k_empty = [&](int s) { return bar0 + 8u * (2 + KS + s); };
  auto v_full = [&](int s) { return bar0 + 8u * (2 + 2 * KS + s); };
  auto v_empty = [&](int s) { return bar0 + 8u * (2 + 2 * KS + VS + s); };
  auto s_full = [&](int g, int sb) { return bar0 + 8u * (2 + 2 * KS + 2 * VS + g * kGroupBars + sb); };
  auto p_full = [&](int g, int sb) { return bar0 + 8u * (2 + 2 * KS + 2 * VS + g * kGroupBars + SB + sb); };
  auto o_done = [&](int g) { return bar0 + 8u * (2 + 2 * KS + 2 * VS + g * kGroupBars + 2 * SB); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
    abort_flag = 0;
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);        // the issuer hands the Q tiles back once the pair's last scores are computed
    for (int s = 0; s < KS; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 1);   // the issuer hands the keys back once every group's scores of the tile are computed
    }
    for (int s = 0; s < VS; ++s) {
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), NG);  // every row group hands the values back (or the issuer does for a group that skips the tile)
    }
    for (int g = 0; g < NG; ++g) {
      for (int sb = 0; sb < SB; ++sb) {
        mbar_init(s_full(g, sb), 1);
        mbar_init(p_full(g, sb), 4);
      }
      mbar_init(o_done(g), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  pdl_launch_dependents();
  pdl_wait();
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"((uint32_t)__cvta_generic_to_shared(&tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_slot;
  auto tmem_s = [&](int g, int sb) { return tmem_base + (uint32_t)g * kGroupCols + (uint32_t)sb * TK; };   // the scores; the weights go over them
  auto tmem_o = [&](int g) { return tmem_base + (uint32_t)g * kGroupCols + SB * TK; };
  volatile int* abortp = &abort_flag;
  const int group = q_heads / kv_heads;
  const int total = items * kv_heads;
  // The pairs are sorted longest first. CTA c takes, in round r, pair r G + c when r is even and r G + (G - 1 - c) when it
  // is odd: the CTA that got the longest pair of one round gets the shortest of the next, so every CTA walks about the
  // same number of tiles. (The last round may leave a CTA without a pair while a later one of the same round has one:
  // the walk then ends for it a round early, which costs it nothing.)
  auto pair_of = [&](int round) { return round * (int)gridDim.x + ((round & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x); };

  // What every thread derives of an (item, head) pair.
  struct Pair {
    int b, row0, kvh, q_start, kv_len, pos0, rows_total;
    int g_first[NG], g_last[NG];  // first and last key tile of each row group (last < first: none)
    int t0, ntiles, lo, hi;
  };
  auto load_pair = [&](int wi, Pair& p) -> bool {
    const int2 w = work[wi / kv_heads];
    p.b = w.x;
    p.row0 = w.y;
    p.kvh = wi % kv_heads;
    if (p.b < 0) return false;  // padding of a fixed-size work list
    p.q_start = q_indptr[p.b];
    const int n = q_indptr[p.b + 1] - p.q_start;
    p.kv_len = kv_lens[p.b];
    p.pos0 = p.kv_len - n;
    p.rows_total = n * group;
    // Key tiles of each row group: from its first row's window to its last row's position; a group past the request's
    // rows has none. The CTA walks the union (the groups' ranges overlap or touch: later rows see later keys).
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      const int r0 = p.row0 + g * BM;
      if (r0 < p.rows_total) {
        const int last_row = min(r0 + BM, p.rows_total) - 1;
        p.g_last[g] = (p.pos0 + last_row / group) / TK;
        p.g_first[g] = (window > 0 ? max(0, p.pos0 + r0 / group - window + 1) : 0) / TK;
      } else {
        p.g_first[g] = 1;
        p.g_last[g] = 0;
      }
    }
    p.t0 = p.g_first[0];
    int t1 = p.g_last[0];
#pragma unroll
    for (int g = 1; g < NG; ++g) {
      if (p.g_last[g] >= p.g_first[g]) t1 = max(t1, p.g_last[g]);
    }
    p.ntiles = t1 - p.t0 + 1;
    p.lo = window > 0 ? max(0, p.pos0 + p.row0 / group - window + 1) : 0;                              // first key any row of the pair sees
    p.hi = min(p.pos0 + (min(p.row0 + NG * BM, p.rows_total) - 1) / group, (t1 + 1) * TK - 1);          // last one
    return p.ntiles > 0;
  };

  if (warp == 0) {
    // ---- producer
    const int page_shift = 31 - __clz(page_size);  // a power of two here
    int kt = 0;        // tiles copied so far, over all pairs: the rings run on
    int pairs = 0;     // pairs begun so far
    bool ok = true;
    Pair p;
    for (int round = 0, wi = pair_of(0); wi < total && ok; wi = pair_of(++round)) {
      if (!load_pair(wi, p)) continue;
      const int32_t* pages = kv_indices + kv_indptr[p.b];
      const int p_first = (p.t0 * TK) >> page_shift, p_last = p.hi >> page_shift;
      const int fallback = pages[p_last];
      auto row_of = [&](int pg, int entry) {  // first pool row of page pg of the request, given its block-table entry
        const bool visible = ((pg + 1) << page_shift) > p.lo && (pg << page_shift) <= p.hi;
        return ((visible && entry >= 0 ? entry : fallback) * kv_heads + p.kvh) << page_shift;
      };
      int batch0 = p_first;
      int cur = row_of(batch0 + lane, batch0 + lane <= p_last ? pages[batch0 + lane] : -1);
      int nxt_entry = batch0 + 32 + lane <= p_last ? pages[batch0 + 32 + lane] : -1;
      if (lane == 0) {
        if (pairs >= 1) ok = mbar_wait_limited(q_empty, (uint32_t)(pairs - 1) & 1u, abortp, 12, &g_attention_tc_error);
        if (ok) {
          mbar_expect_tx(q_full, NG * kQBytes);  // rows past the tensor's last token are filled with zeros and counted
#pragma unroll
          for (int g = 0; g < NG; ++g) tma_load_5d(q_smem + g * kQBytes, &map_q, q_full, 0, 0, p.kvh, p.q_start + (p.row0 + g * BM) / group, 0);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      ++pairs;
      for (int i = 0; i < p.ntiles && ok; ++i, ++kt) {
        const int ks = kt % KS, vs = kt % VS;
        const int j = (p.t0 + i) * TK;
        if ((j >> page_shift) >= batch0 + 32) {  // uniform in the warp
          batch0 += 32;
          cur = row_of(batch0 + lane, nxt_entry);
          nxt_entry = batch0 + 32 + lane <= p_last ? pages[batch0 + 32 + lane] : -1;
        }
        // lane L issues copy L of the tile: page copy L / (CB + 1); column block L % (CB + 1) of its keys, or its values.
        // A tile never straddles two batches of 32 pages: both start on tile boundaries.
        const int c = lane / (CB + 1), part = lane % (CB + 1);
        const int jc = j + (c < NP ? c : 0) * RPC;
        const int my_row = __shfl_sync(0xffffffffu, cur, ((jc >> page_shift) - batch0) & 31) + (jc & (page_size - 1));
        if (lane == 0) {
          if (kt >= KS) ok = mbar_wait_limited(k_empty(ks), (uint32_t)((kt / KS) - 1) & 1u, abortp, 1, &g_attention_tc_error);
          if (ok) mbar_expect_tx(k_full(ks), kTile);
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;  // also orders the expected bytes before the copies
        if (ok && lane < kOps && part < CB) {
          tma_load_2d(k_smem + ks * kTile + part * (TK * 128) + c * (RPC * 128), &map_k, k_full(ks), part * 64, my_row);
        }
        if (lane == 0 && ok) {
          if (kt >= VS) ok = mbar_wait_limited(v_empty(vs), (uint32_t)((kt / VS) - 1) & 1u, abortp, 9, &g_attention_tc_error);
          if (ok) mbar_expect_tx(v_full(vs), kTile);
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (ok && lane < kOps && part == CB) {
          tma_load_3d(v_smem + vs * kTile + c * kVPage, &map_v, v_full(vs), 0, my_row, 0);
        }
      }
    }
  } else if (warp == 1) {
    // ---- issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(BM, TK);
      constexpr uint32_t idesc_o = umma_idesc_bf16_b_mn(BM, D);
      int kt0 = 0;            // tiles of the pairs before this one
      int pairs = 0;
      int jt0[NG];            // tiles of each group in the pairs before this one: which score columns, which phase
#pragma unroll
      for (int g = 0; g < NG; ++g) jt0[g] = 0;
      bool ok = true;
      Pair p;
      for (int round = 0, wi = pair_of(0); wi < total && ok; wi = pair_of(++round)) {
        if (!load_pair(wi, p)) continue;
        if (!(ok = mbar_wait_limited(q_full, (uint32_t)pairs & 1u, abortp, 2, &g_attention_tc_error))) break;
        ++pairs;
        tcgen05_fence_after();
        // O_g += P V of the pair's tile i (the group's tile j): the weights from tensor memory, the values from the ring
        auto issue_pv = [&](int g, int j, int i) {
          const int jt = jt0[g] + j, sb = jt % SB;
          if (!(ok = mbar_wait_limited(p_full(g, sb), (uint32_t)(jt / SB) & 1u, abortp, 3, &g_attention_tc_error))) return;
          tcgen05_fence_after();
          const uint32_t v0 = v_smem + ((kt0 + i) % VS) * kTile;
#pragma unroll
          for (int kk = 0; kk < TK / 16; ++kk) {
            const uint32_t v_rows = v0 + (uint32_t)((kk * 16) / RPC) * kVPage + (uint32_t)((kk * 16) % RPC) * 128;
            const uint64_t b_desc = umma_desc_mn_major_sw128(v_rows, RPC * 128, 1024);
            tcgen05_mma_f16_ts(tmem_o(g), tmem_s(g, sb) + (uint32_t)(kk * 8), b_desc, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
          }
          tcgen05_commit(v_empty((kt0 + i) % VS));  // the values are free (for this group) once these products have read them
          if (p.g_first[g] + j == p.g_last[g]) tcgen05_commit(o_done(g));
        };
        // S_g = Q K^T of the pair's tile i
        auto issue_s = [&](int g, int j, int i) {
          const int jt = jt0[g] + j;
          const uint32_t k0 = k_smem + ((kt0 + i) % KS) * kTile;
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint64_t a_desc = umma_desc_k_major_sw128(q_smem + g * kQBytes + (k / 4) * (BM * 128)) + (uint64_t)(2 * (k % 4));
            const uint64_t b_desc = umma_desc_k_major_sw128(k0 + (k / 4) * (TK * 128)) + (uint64_t)(2 * (k % 4));
            tcgen05_mma_f16(tmem_s(g, jt % SB), a_desc, b_desc, idesc_s, k > 0 ? 1u : 0u);
          }
          tcgen05_commit(s_full(g, jt % SB));
        };
        for (int i = 0; i <= p.ntiles && ok; ++i) {
          const int t = p.t0 + i;
          if (i < p.ntiles) {
            if (!(ok = mbar_wait_limited(k_full((kt0 + i) % KS), (uint32_t)((kt0 + i) / KS) & 1u, abortp, 4, &g_attention_tc_error))) break;
            tcgen05_fence_after();
          }
          if (SB == 2 && i < p.ntiles) {
            // two sets of score columns: this tile's scores are computed while the softmax of the tile before still runs.
            // (The set they go to held the weights of the group's tile two before, whose second product was issued an
            // iteration ago.)
#pragma unroll
            for (int g = 0; g < NG; ++g)
              if (t >= p.g_first[g] && t <= p.g_last[g]) issue_s(g, t - p.g_first[g], i);
          }
          if (i >= 1) {
            if (!(ok = mbar_wait_limited(v_full((kt0 + i - 1) % VS), (uint32_t)((kt0 + i - 1) / VS) & 1u, abortp, 5, &g_attention_tc_error))) break;
            tcgen05_fence_after();
          }
#pragma unroll
          for (int g = 0; g < NG; ++g) {
            if (i >= 1) {   // the second product of the tile before, which the group's softmax has finished meanwhile
              if (t - 1 >= p.g_first[g] && t - 1 <= p.g_last[g]) {
                issue_pv(g, t - 1 - p.g_first[g], i - 1);
                if (!ok) break;
              } else {
                mbar_arrive(v_empty((kt0 + i - 1) % VS));
              }
            }
            // one set of score columns: the scores overwrite the weights the product just issued reads (in issue order)
            if (SB == 1 && i < p.ntiles && t >= p.g_first[g] && t <= p.g_last[g]) issue_s(g, t - p.g_first[g], i);
          }
          if (ok && i < p.ntiles) tcgen05_commit(k_empty((kt0 + i) % KS));
          if (ok && i == p.ntiles - 1) tcgen05_commit(q_empty);   // the pair's last scores are on their way: Q may be replaced
        }
        kt0 += p.ntiles;
#pragma unroll
        for (int g = 0; g < NG; ++g) jt0[g] += max(0, p.g_last[g] - p.g_first[g] + 1);
      }
    }
  } else {
    // ---- softmax, correction, epilogue: one thread a row, four warps a row group
    const int g = (warp - 2) / 4;
    const int lane_group = warp & 3;               // the tensor-memory lanes this warp may touch
    const int row = lane_group * 32 + lane;        // row within the group
    const uint32_t lane_addr = (uint32_t)(lane_group * 32) << 16;
    const int tid_g = threadIdx.x - 64 - g * kGroupThreads;     // 0 .. 127 within the group
    int kt0 = 0;        // tiles of the pairs before this one (the rings' positions)
    int jt0 = 0;        // this group's tiles in the pairs before this one
    int outs = 0;       // pairs in which this group had rows: the phase of o_done
    bool ok = true;
    Pair p;
    for (int round = 0, wi = pair_of(0); wi < total && ok; wi = pair_of(++round)) {
      if (!load_pair(wi, p)) continue;
      const int pr = p.row0 + g * BM + row;
      const bool valid = pr < p.rows_total;
      const int qpos = valid ? p.pos0 + pr / group : -1;
      const int qlo = valid && window > 0 ? max(0, qpos - window + 1) : 0;
      const int my_tiles = p.g_last[g] - p.g_first[g] + 1;  // at most 0 for a group without rows
      float m = -INFINITY, l = 0.f;
      for (int j = 0; j < my_tiles && ok; ++j) {
        const int i = p.g_first[g] + j - p.t0;       // the pair's tile
        const int kt = kt0 + i;
        const int jt = jt0 + j, sb = jt % SB;
        const int j0 = (p.g_first[g] + j) * TK;
        if (!(ok = mbar_wait_limited(s_full(g, sb), (uint32_t)(jt / SB) & 1u, abortp, 6, &g_attention_tc_error))) break;
        tcgen05_fence_after();
        float s[TK];
        {
          uint32_t v[TK / 32][32];
#pragma unroll
          for (int c = 0; c < TK / 32; ++c) tcgen05_ld_32x32b_x32_nowait(tmem_s(g, sb) + lane_addr + c * 32, v[c]);
          tcgen05_wait_ld();
#pragma unroll
          for (int c = 0; c < TK / 32; ++c)
#pragma unroll
            for (int e = 0; e < 32; ++e) s[c * 32 + e] = __uint_as_float(v[c][e]);
        }
        if (!(j0 + TK - 1 <= qpos && j0 >= qlo)) {
#pragma unroll
          for (int e = 0; e < TK; ++e) {
            const int key = j0 + e;
            s[e] = (key <= qpos && key >= qlo) ? s[e] : -INFINITY;
          }
        }
        // the maximum of the raw scores (the scale is positive); four chains, so that it is not one long dependency
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < TK; e += 4) {
#pragma unroll
          for (int u = 0; u < 4; ++u) mx4[u] = fmaxf(mx4[u], s[e + u]);
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
        // the reference maximum moves only when it must: the weights of this tile are then at most 2^kTcLazyRescale
        float corr = 1.0f;
        if (mx > m + kTcLazyRescale || (m == -INFINITY && mx > -INFINITY)) {
          corr = ex2(m - mx);   // 0 when m is -inf
          m = mx;
        }
        const float msafe = m == -INFINITY ? 0.f : m;  // a row that has seen no key yet: every weight below is 0
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t packed[TK / 2];
#pragma unroll
        for (int e = 0; e < TK; e += 2) {
          const float p0 = ex2(fmaf(s[e], scale_log2, -msafe)), p1 = ex2(fmaf(s[e + 1], scale_log2, -msafe));
          sum4[(e / 2) & 3] += p0 + p1;
          __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
          packed[e / 2] = *reinterpret_cast<uint32_t*>(&pb);
        }
        l = l * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        // The accumulator holds the pair's tiles 0 .. j - 1 once the second product of tile j - 1 is done. With one set
        // of score columns the scores of tile j were computed after it (the issuer's order). With two sets they were
        // issued before it: the group then waits for that product where it hands the values back.
        if (j >= 1 && __any_sync(0xffffffffu, corr != 1.0f)) {
          if (SB == 2) {
            if (!(ok = mbar_wait_limited(v_empty((kt - 1) % VS), (uint32_t)((kt - 1) / VS) & 1u, abortp, 10, &g_attention_tc_error))) break;
            tcgen05_fence_after();
          }
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t v[32];
            tcgen05_ld_32x32b_x32(tmem_o(g) + lane_addr + c * 32, v);
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * corr);
            tcgen05_st_32x32b_x32(tmem_o(g) + lane_addr + c * 32, v);
          }
        }
        // value rows at positions the request does not hold yet, and rows before the first visible key (their page may
        // have been given back and replaced by another): zero, once the tile's values have landed. Every row group does
        // it before its own second product.
        if (j0 + TK > p.kv_len || j0 < p.lo) {
          if (!(ok = mbar_wait_limited(v_full(kt % VS), (uint32_t)(kt / VS) & 1u, abortp, 7, &g_attention_tc_error))) break;
          const uint32_t v0 = v_smem + (kt % VS) * kTile;
          for (int idx = tid_g; idx < TK * (D / 8); idx += kGroupThreads) {
            const int r = idx / (D / 8), ch = idx % (D / 8);
            if (j0 + r >= p.kv_len || j0 + r < p.lo) {
              const uint32_t addr = v0 + (uint32_t)(r / RPC) * kVPage + (uint32_t)(ch >> 3) * (RPC * 128) + (uint32_t)(r % RPC) * 128 +
                                    (uint32_t)(((ch & 7) ^ (r & 7)) << 4);
              asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(addr), "r"(0u) : "memory");
            }
          }
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // the stores are visible to the tensor cores' reads
        }
        // the row's weights, two bfloat16 a column, over the first half of the scores' columns
#pragma unroll
        for (int c = 0; c < TK / 64; ++c) tcgen05_st_32x32b_x32_nowait(tmem_s(g, sb) + lane_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&packed[c * 32]));
        tcgen05_wait_st();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full(g, sb));
      }
      // epilogue: O / l
      if (ok && my_tiles > 0) ok = mbar_wait_limited(o_done(g), (uint32_t)outs & 1u, abortp, 8, &g_attention_tc_error);
      if (ok && my_tiles > 0) {
        tcgen05_fence_after();
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        __nv_bfloat16* dst = valid ? out + ((size_t)(p.q_start + pr / group) * q_heads + p.kvh * group + pr % group) * D : nullptr;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          tcgen05_ld_32x32b_x32(tmem_o(g) + lane_addr + c * 32, v);
          if (valid) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              uint32_t o[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                __nv_bfloat162 ob = __floats2bfloat162_rn(__uint_as_float(v[e + 2 * u]) * inv, __uint_as_float(v[e + 2 * u + 1]) * inv);
                o[u] = *reinterpret_cast<uint32_t*>(&ob);
              }
              *reinterpret_cast<uint4*>(dst + c * 32 + e) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
        }
        // the accumulator's columns are read: only now may this warp's arrival for the next pair's first weights come
        tcgen05_fence_before();
      }
      if (my_tiles > 0) {
        ++outs;
        jt0 += my_tiles;
      }
      kt0 += p.ntiles;
    }
  }

  __syncwarp();
  if (*abortp) {  // copies in flight land before shared memory is released
    const long long c0 = clock64();
    while (clock64() - c0 < 2000000LL) __nanosleep(256);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ host side
static bool g_prefill_tc = true;

bool prefill_tc_serves(int head_dim, int q_heads, int kv_heads, int page_size, long long pool_pages, const void* k_pool, const void* v_pool,
                       const void* q) {
  if (!g_prefill_tc || pool_pages <= 0 || (head_dim != 64 && head_dim != 128) || kv_heads <= 0 || q_heads % kv_heads != 0) return false;
  const int group = q_heads / kv_heads;
  if (group > 128 || (group & (group - 1)) != 0) return false;  // a CTA's 128 packed rows are whole tokens
  if (page_size < 16 || (page_size & (page_size - 1)) != 0) return false;
  if (pool_pages * kv_heads * page_size >= (1LL << 31)) return false;
  const long long pool_bytes = pool_pages * kv_heads * page_size * head_dim * 2;
  const long long gap = (const char*)v_pool - (const char*)k_pool;
  if (gap < pool_bytes || gap % 16 != 0 || gap >= (1LL << 40)) return false;
  return (uintptr_t)k_pool % 128 == 0 && (q == nullptr || (uintptr_t)q % 16 == 0) && encode_tiled() != nullptr;
}

template <int D, int RPC, int NG>
static int launch_tc(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* out, const int32_t* q_indptr, const int32_t* kv_lens,
                     const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work, int items, int q_heads, int kv_heads,
                     int page_size, float scale, int window, cudaStream_t s) {
  constexpr size_t smem = TcCfg<D, NG>::kSmem;
  auto kernel = attention_prefill_tc_kernel<D, RPC, NG>;
  static int sms[64] = {};   // per device: its SM count, and that the kernel's shared-memory size has been set there
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return fail(ROOST_ERR_UNSUPPORTED, "attention_prefill: device ordinal beyond 63");
  if (sms[dev] == 0) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
  }
  // One CTA fills an SM (shared memory, tensor memory). With a few pairs an SM the grid is persistent, one CTA an SM,
  // each walking its share of the sorted list (measured at 1 x 2048 tokens of 32/8 heads: 50 against 72 us); with many
  // pairs an SM every pair is a CTA of its own and the hardware hands them out as SMs fall free, which balances a long
  // list better than the fixed walk (8 x 8192 tokens: 1017 against 885 TFLOP/s).
  const long long pairs = (long long)items * kv_heads;
  const int grid = (int)(pairs <= 8LL * sms[dev] ? (pairs < sms[dev] ? pairs : sms[dev]) : pairs);
  launch_kernel(kernel, dim3(grid), dim3(64 + NG * 128), smem, s, mq, mk, mv, (__nv_bfloat16*)out, q_indptr, kv_lens, kv_indptr, kv_indices,
                (const int2*)work, items, q_heads, kv_heads, page_size, scale * kLog2eTc, window);
  return check_launch("attention_prefill_tc");
}

int launch_prefill_tc(const void* q, long long tokens, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr,
                      const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work, int items, int tile_rows,
                      int q_heads, int kv_heads, int head_dim, int page_size, long long pool_pages, float scale, int window, cudaStream_t s) {
  if (tile_rows != 128 && tile_rows != 256) return fail(ROOST_ERR_INVALID, "attention_prefill: the tcgen05 kernel takes work items of 128 or 256 packed rows");
  const int groups = tile_rows / kTcRows;
  const int group = q_heads / kv_heads;
  CUtensorMap mq;
  {
    // q [tokens][kv_heads][group][D] as 64 columns x group x kv heads x tokens x column blocks; a box is 128 packed rows
    // of one key/value head: [column block][token][head of the group][64]
    const cuuint64_t dims[5] = {64u, (cuuint64_t)group, (cuuint64_t)kv_heads, (cuuint64_t)tokens, (cuuint64_t)head_dim / 64};
    const cuuint64_t strides[4] = {(cuuint64_t)head_dim * 2, (cuuint64_t)group * head_dim * 2, (cuuint64_t)q_heads * head_dim * 2, 128u};
    const cuuint32_t box[5] = {64u, (cuuint32_t)group, 1u, (cuuint32_t)(kTcRows / group), (cuuint32_t)head_dim / 64};
    const cuuint32_t elem[5] = {1, 1, 1, 1, 1};
    const CUresult r = encode_tiled()(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(q), dims, strides, box, elem,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ROOST_ERR_CUDA, "attention_prefill: cuTensorMapEncodeTiled (q) failed with code " + std::to_string((int)r));
  }
  const int box_rows = page_size < 32 ? page_size : 32;
  const cuuint64_t pool_rows = (cuuint64_t)(pool_pages * kv_heads * page_size);
  CUtensorMap mk, mv;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)head_dim, pool_rows};
    const cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode_tiled()(&mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(k_pool), dims, strides, box, elem,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ROOST_ERR_CUDA, "attention_prefill: cuTensorMapEncodeTiled (keys) failed with code " + std::to_string((int)r));
  }
  {
    const cuuint64_t dims[3] = {64u, pool_rows, (cuuint64_t)head_dim / 64};
    const cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2, 128u};
    const cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, (cuuint32_t)head_dim / 64};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult r = encode_tiled()(&mv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(v_pool), dims, strides, box, elem,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ROOST_ERR_CUDA, "attention_prefill: cuTensorMapEncodeTiled (values) failed with code " + std::to_string((int)r));
  }
#define ROOST_TC_CASE(DD, RR, GG)                                                                                                      \
  if (head_dim == DD && box_rows == RR && groups == GG)                                                                                \
    return launch_tc<DD, RR, GG>(mq, mk, mv, out, q_indptr, kv_lens, kv_indptr, kv_indices, work, items, q_heads, kv_heads, page_size, \
                                 scale, window, s);
  ROOST_TC_CASE(128, 16, 1)
  ROOST_TC_CASE(128, 32, 1)
  ROOST_TC_CASE(64, 16, 1)
  ROOST_TC_CASE(64, 32, 1)
  ROOST_TC_CASE(128, 16, 2)
  ROOST_TC_CASE(128, 32, 2)
  ROOST_TC_CASE(64, 16, 2)
  ROOST_TC_CASE(64, 32, 2)
#undef ROOST_TC_CASE
  return fail(ROOST_ERR_UNSUPPORTED, "attention_prefill: no tcgen05 kernel for these sizes");
}

void set_prefill_tc(bool on) { g_prefill_tc = on; }

int* attention_tc_error_address() {
  int* p = nullptr;
  return cudaGetSymbolAddress((void**)&p, g_attention_tc_error) == cudaSuccess ? p : nullptr;
}

int prefill_tc_status() {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_attention_tc_error, sizeof(int)) != cudaSuccess) return -1;
  if (code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_attention_tc_error, &zero, sizeof(int));
  }
  return code;
}

}  // namespace roost

ROOST_TRACE_TU(attention_tc)
