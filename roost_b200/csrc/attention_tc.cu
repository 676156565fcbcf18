// Causal grouped-query attention over the paged cache for prompt portions (rows with more than 16 packed rows), on the
// fifth-generation tensor cores: both products are tcgen05.mma with the accumulators in tensor memory.
//
// Definition and numerics as in attention_mma.cu (src/Starlings.Roost.Ops/CpuOps.cs:181-298; 32-bit scores, maxima,
// exponentials, sums and output accumulation; the softmax weights rounded to bfloat16 as the operand of the second
// product, kernels/README.md:234-236). A CTA owns 128 packed rows (token r / G, head r % G) of one request and one
// key/value head and walks the keys in tiles of 64 at fixed absolute positions, so a row's bits do not depend on how
// the prompt was cut or on what else is in the batch.
//   warp 0 (producer): one 5-D tensor copy brings the Q tile [128 rows x D] into 128-byte-swizzled shared memory; per key
//     tile it looks the pages up and its lanes issue the stage's copies side by side: per page one copy per 64-column
//     block of the keys, placed so that the tile's 64 key rows are consecutive in each block (one product then takes
//     them all), and one copy of the values.
//   warp 1 (issuer, one lane): S = Q K^T (M 128, N 64, K = D) into one of two score buffers in tensor memory; O += P V, one product per 16 keys (M 128, N = D, K 16) with P from shared
//     memory and V as the N-major operand exactly as the copy left it. tcgen05.commit tells the others when the scores
//     are there, when a stage is free and when the output accumulator has taken a tile in.
//   warps 2..5 (softmax, one thread a row): read the row's 64 scores from tensor memory, scale, mask by position, keep
//     the running maximum and sum, rescale the row of the output accumulator in tensor memory when the maximum moved
//     (skipped when no row of the warp moved), write the weights as bfloat16 into the swizzled P tile, and at the end
//     divide the accumulator by the sum and write the row out.
// The scores of tile j + 1 are computed while the softmax of tile j runs. Value rows at positions the request does not
// hold yet (the rest of its last page) or before the CTA's first visible key are zeroed in shared memory before the second product, so that whatever the pool
// holds there cannot reach a result; their scores are masked by position. Every wait is bounded (see tma.cuh): a wait
// given up raises the CTA's abort flag and records a code that roost_attention_status() returns.
#include "tcgen05.cuh"

namespace roost {

constexpr float kLog2eTc = 1.4426950408889634f;
constexpr int kTcRows = 128;   // packed rows of a CTA
constexpr int kTcKeys = 64;    // keys of a tile
__device__ int g_attention_tc_error = 0;

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3, int c4) {
  asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];\n" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
               : "memory");
}

// 2^x in one special-function instruction (inputs here are at most 0 or -inf; results below 2^-126 flush to zero)
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

template <int D, int NG>
constexpr int tc_stages() {  // what fits beside NG Q tiles and NG P tiles in 227 KB
  return D == 128 ? (NG == 1 ? 4 : 3) : 6;
}

// work[i] = (batch row, first packed row of the CTA's NG x 128 rows)
template <int D, int RPC, int NG>
__global__ void __launch_bounds__(64 + NG * 128, 1)
    attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ q_indptr,
                                const int32_t* __restrict__ kv_lens, const int32_t* __restrict__ kv_indptr,
                                const int32_t* __restrict__ kv_indices, const int2* __restrict__ work, int q_heads, int kv_heads, int page_size,
                                float scale_log2, int window) {
  constexpr int BM = kTcRows, TK = kTcKeys, STAGES = tc_stages<D, NG>(), NP = TK / RPC, CB = D / 64;
  constexpr uint32_t kQBytes = BM * D * 2;                  // one row group's Q tile
  constexpr uint32_t kStageBytes = 2 * TK * D * 2;          // keys and values of TK positions
  constexpr uint32_t kKeys = TK * D * 2;                    // a stage's keys: [column block][TK rows][128 B], K-major for one product
  constexpr uint32_t kVPage = CB * RPC * 128;               // its values, page copy by page copy: [column block][RPC rows][128 B]
  constexpr int kOps = NP * (CB + 1);                       // copies a stage takes: per page one per column block of keys, one of values
  static_assert(kOps <= 32, "one lane a copy");
  constexpr uint32_t kPBytes = BM * 128;                    // a row group's P tile: 128 rows x 64 keys of bfloat16
  constexpr uint32_t kGroupCols = 2 * TK + D;               // tensor-memory columns of a row group: two score buffers and the output
  constexpr uint32_t kTmemCols = NG * kGroupCols <= 256 ? 256 : 512;
  static_assert(NG * kGroupCols <= 512, "tensor memory has 512 columns");
  constexpr int kGroupBars = 8;                             // s_full[2], s_empty[2], p_full[2], pv_done[2]
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = ((uint32_t)__cvta_generic_to_shared(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;
  const uint32_t kv_smem = q_smem + NG * kQBytes;
  const uint32_t p_smem = kv_smem + STAGES * kStageBytes;
  __shared__ __align__(8) uint64_t bars[1 + 2 * STAGES + NG * kGroupBars];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(bars);
  const uint32_t q_full = bar0;
  auto kv_full = [&](int s) { return bar0 + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bar0 + 8u * (1 + STAGES + s); };
  auto s_full = [&](int g, int i) { return bar0 + 8u * (1 + 2 * STAGES + g * kGroupBars + i); };
  auto s_empty = [&](int g, int i) { return bar0 + 8u * (1 + 2 * STAGES + g * kGroupBars + 2 + i); };
  auto p_full = [&](int g, int i) { return bar0 + 8u * (1 + 2 * STAGES + g * kGroupBars + 4 + i); };
  auto pv_done = [&](int g, int i) { return bar0 + 8u * (1 + 2 * STAGES + g * kGroupBars + 6 + i); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
    abort_flag = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), NG);  // every row group hands the stage back (or the issuer does for a group that skips the tile)
    }
    for (int g = 0; g < NG; ++g) {
      for (int i = 0; i < 2; ++i) {
        mbar_init(s_full(g, i), 1);
        mbar_init(s_empty(g, i), 4);
        mbar_init(p_full(g, i), 4);
        mbar_init(pv_done(g, i), 1);
      }
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  pdl_launch_dependents();
  pdl_wait();
  const int2 w = work[blockIdx.x];
  const int b = w.x, row0 = w.y;
  if (b < 0) return;  // padding of a fixed-size work list (before anything is allocated)
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
  auto tmem_s = [&](int g, int i) { return tmem_base + (uint32_t)g * kGroupCols + (uint32_t)i * TK; };
  auto tmem_o = [&](int g) { return tmem_base + (uint32_t)g * kGroupCols + 2 * TK; };
  volatile int* abortp = &abort_flag;

  const int kvh = blockIdx.y;
  const int group = q_heads / kv_heads;
  const int q_start = q_indptr[b];
  const int n = q_indptr[b + 1] - q_start;
  const int kv_len = kv_lens[b];
  const int pos0 = kv_len - n;
  const int rows_total = n * group;
  // Key tiles of each row group: from its first row's window to its last row's position; a group past the request's
  // rows has none. The CTA walks the union (the groups' ranges overlap or touch: later rows see later keys).
  int g_first[NG], g_last[NG];  // first and last key tile of the group (last < first: none)
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    const int r0 = row0 + g * BM;
    if (r0 < rows_total) {
      const int last_row = min(r0 + BM, rows_total) - 1;
      g_last[g] = (pos0 + last_row / group) / TK;
      g_first[g] = (window > 0 ? max(0, pos0 + r0 / group - window + 1) : 0) / TK;
    } else {
      g_first[g] = 1;
      g_last[g] = 0;
    }
  }
  int t0 = g_first[0], t1 = g_last[0];
#pragma unroll
  for (int g = 1; g < NG; ++g) {
    if (g_last[g] >= g_first[g]) t1 = max(t1, g_last[g]);
  }
  const int ntiles = t1 - t0 + 1;
  const int lo = window > 0 ? max(0, pos0 + row0 / group - window + 1) : 0;                    // first key any row of the CTA sees
  const int hi = min(pos0 + (min(row0 + NG * BM, rows_total) - 1) / group, (t1 + 1) * TK - 1);  // last one

  if (warp == 0) {
    // ---- producer
    const int page_shift = 31 - __clz(page_size);  // a power of two here
    const int32_t* pages = kv_indices + kv_indptr[b];
    const int p_first = (t0 * TK) >> page_shift, p_last = hi >> page_shift;
    const int fallback = pages[p_last];
    auto row_of = [&](int p, int entry) {  // first pool row of page p of the request, given its block-table entry
      const bool visible = ((p + 1) << page_shift) > lo && (p << page_shift) <= hi;
      return ((visible && entry >= 0 ? entry : fallback) * kv_heads + kvh) << page_shift;
    };
    int batch0 = p_first;
    int cur = row_of(batch0 + lane, batch0 + lane <= p_last ? pages[batch0 + lane] : -1);
    int nxt_entry = batch0 + 32 + lane <= p_last ? pages[batch0 + 32 + lane] : -1;
    if (lane == 0) {
      mbar_expect_tx(q_full, NG * kQBytes);  // rows past the tensor's last token are filled with zeros and counted
#pragma unroll
      for (int g = 0; g < NG; ++g) tma_load_5d(q_smem + g * kQBytes, &map_q, q_full, 0, 0, kvh, q_start + (row0 + g * BM) / group, 0);
    }
    bool ok = true;
    for (int i = 0; i < ntiles && ok; ++i) {
      const int stage = i % STAGES;
      const uint32_t dst = kv_smem + stage * kStageBytes;
      const int j = (t0 + i) * TK;
      if ((j >> page_shift) >= batch0 + 32) {  // uniform in the warp
        batch0 += 32;
        cur = row_of(batch0 + lane, nxt_entry);
        nxt_entry = batch0 + 32 + lane <= p_last ? pages[batch0 + 32 + lane] : -1;
      }
      // lane L issues copy L of the stage: page copy L / (CB + 1); column block L % (CB + 1) of its keys, or its values.
      // A tile never straddles two batches of 32 pages: both start on tile boundaries.
      const int c = lane / (CB + 1), part = lane % (CB + 1);
      const int jc = j + (c < NP ? c : 0) * RPC;
      const int my_row = __shfl_sync(0xffffffffu, cur, ((jc >> page_shift) - batch0) & 31) + (jc & (page_size - 1));
      if (lane == 0) {
        if (i >= STAGES) ok = mbar_wait_limited(kv_empty(stage), (uint32_t)((i / STAGES) - 1) & 1u, abortp, 1, &g_attention_tc_error);
        if (ok) mbar_expect_tx(kv_full(stage), kStageBytes);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;  // also orders the expected bytes before the copies
      if (ok && lane < kOps) {
        if (part < CB) {
          tma_load_2d(dst + part * (TK * 128) + c * (RPC * 128), &map_k, kv_full(stage), part * 64, my_row);
        } else {
          tma_load_3d(dst + kKeys + c * kVPage, &map_v, kv_full(stage), 0, my_row, 0);
        }
      }
    }
  } else if (warp == 1) {
    // ---- issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(BM, TK);
      constexpr uint32_t idesc_o = umma_idesc_bf16_b_mn(BM, D);
      bool ok = mbar_wait_limited(q_full, 0, abortp, 2, &g_attention_tc_error);
      tcgen05_fence_after();
      // O_g += P V of the group's tile number j (the CTA's tile i): after it the stage is the group's no longer
      auto issue_pv = [&](int g, int j, int i) {
        const int stage = i % STAGES;
        if (!(ok = mbar_wait_limited(p_full(g, j & 1), (uint32_t)(j >> 1) & 1u, abortp, 3, &g_attention_tc_error))) return;
        tcgen05_fence_after();
        const uint32_t v0 = kv_smem + stage * kStageBytes + kKeys;
#pragma unroll
        for (int kk = 0; kk < TK / 16; ++kk) {
          const uint32_t v_rows = v0 + (uint32_t)((kk * 16) / RPC) * kVPage + (uint32_t)((kk * 16) % RPC) * 128;
          const uint64_t a_desc = umma_desc_k_major_sw128(p_smem + g * kPBytes) + (uint64_t)(2 * kk);
          const uint64_t b_desc = umma_desc_mn_major_sw128(v_rows, RPC * 128, 1024);
          tcgen05_mma_f16(tmem_o(g), a_desc, b_desc, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
        tcgen05_commit(kv_empty(stage));  // the stage is free (for this group) once these products have read it
        tcgen05_commit(pv_done(g, j & 1));
      };
      // the second product of tile i for every group that has it; a group without it gives the stage back at once
      auto finish_tile = [&](int i) {
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          const int t = t0 + i;
          if (t >= g_first[g] && t <= g_last[g]) {
            if (ok) issue_pv(g, t - g_first[g], i);
          } else {
            mbar_arrive(kv_empty(i % STAGES));
          }
        }
      };
      for (int i = 0; i < ntiles && ok; ++i) {
        const int stage = i % STAGES, t = t0 + i;
        if (!(ok = mbar_wait_limited(kv_full(stage), (uint32_t)(i / STAGES) & 1u, abortp, 4, &g_attention_tc_error))) break;
        tcgen05_fence_after();
        const uint32_t k0 = kv_smem + stage * kStageBytes;
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          if (t < g_first[g] || t > g_last[g]) continue;
          const int j = t - g_first[g];
          if (j >= 2 && !(ok = mbar_wait_limited(s_empty(g, j & 1), (uint32_t)((j >> 1) - 1) & 1u, abortp, 5, &g_attention_tc_error))) break;
          tcgen05_fence_after();
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint64_t a_desc = umma_desc_k_major_sw128(q_smem + g * kQBytes + (k / 4) * (BM * 128)) + (uint64_t)(2 * (k % 4));
            const uint64_t b_desc = umma_desc_k_major_sw128(k0 + (k / 4) * (TK * 128)) + (uint64_t)(2 * (k % 4));
            tcgen05_mma_f16(tmem_s(g, j & 1), a_desc, b_desc, idesc_s, k > 0 ? 1u : 0u);
          }
          tcgen05_commit(s_full(g, j & 1));
        }
        if (ok && i >= 1) finish_tile(i - 1);
      }
      if (ok && ntiles > 0) finish_tile(ntiles - 1);
    }
  } else {
    // ---- softmax, correction, epilogue: one thread a row, four warps a row group
    const int g = (warp - 2) / 4;
    const int lane_group = warp & 3;               // the tensor-memory lanes this warp may touch
    const int row = lane_group * 32 + lane;        // row within the group
    const int pr = row0 + g * BM + row;
    const bool valid = pr < rows_total;
    const int qpos = valid ? pos0 + pr / group : -1;
    const int qlo = valid && window > 0 ? max(0, qpos - window + 1) : 0;
    const uint32_t lane_addr = (uint32_t)(lane_group * 32) << 16;
    const int my_tiles = g_last[g] - g_first[g] + 1;  // at most 0 for a group without rows
    const int tid_g = threadIdx.x - 64 - g * 128;     // 0 .. 127 within the group
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < my_tiles && ok; ++j) {
      const int stage = (g_first[g] + j - t0) % STAGES;
      const int j0 = (g_first[g] + j) * TK;
      if (!(ok = mbar_wait_limited(s_full(g, j & 1), (uint32_t)(j >> 1) & 1u, abortp, 6, &g_attention_tc_error))) break;
      tcgen05_fence_after();
      float s[TK];
      {
        uint32_t v[TK / 32][32];
#pragma unroll
        for (int c = 0; c < TK / 32; ++c) tcgen05_ld_32x32b_x32_nowait(tmem_s(g, j & 1) + lane_addr + c * 32, v[c]);
        tcgen05_wait_ld();
#pragma unroll
        for (int c = 0; c < TK / 32; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(v[c][i]);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty(g, j & 1));  // the scores are in registers: the buffer may take tile j + 2
      if (!(j0 + TK - 1 <= qpos && j0 >= qlo)) {
#pragma unroll
        for (int i = 0; i < TK; ++i) {
          const int key = j0 + i;
          s[i] = (key <= qpos && key >= qlo) ? s[i] : -INFINITY;
        }
      }
      // the maximum of the raw scores (the scale is positive); four chains, so that it is not one long dependency
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < TK; i += 4) {
#pragma unroll
        for (int e = 0; e < 4; ++e) mx4[e] = fmaxf(mx4[e], s[i + e]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m, mx * scale_log2);
      const float msafe = m_new == -INFINITY ? 0.f : m_new;  // a row that has seen no key yet: every weight below is 0
      const float corr = ex2(m - msafe);                       // 0 when m is -inf
      m = m_new;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t packed[TK / 2];
#pragma unroll
      for (int i = 0; i < TK; i += 2) {
        const float p0 = ex2(fmaf(s[i], scale_log2, -msafe)), p1 = ex2(fmaf(s[i + 1], scale_log2, -msafe));
        sum4[(i / 2) & 3] += p0 + p1;
        __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
        packed[i / 2] = *reinterpret_cast<uint32_t*>(&pb);
      }
      l = l * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      // the accumulator holds tiles 0 .. j - 1 once the product of tile j - 1 is done; then its row may be rescaled
      // and the P tile (which that product read) written again
      if (j >= 1 && !(ok = mbar_wait_limited(pv_done(g, (j - 1) & 1), (uint32_t)((j - 1) >> 1) & 1u, abortp, 7, &g_attention_tc_error))) break;
      tcgen05_fence_after();
      if (j >= 1 && __any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          tcgen05_ld_32x32b_x32(tmem_o(g) + lane_addr + c * 32, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
          tcgen05_st_32x32b_x32(tmem_o(g) + lane_addr + c * 32, v);
        }
      }
      // value rows at positions the request does not hold yet, and rows before the first visible key (their page may
      // have been given back and replaced by another): zero (the copies of this stage have landed: the scores of this
      // tile were computed from the same stage). Every row group does it before its own second product.
      if (j0 + TK > kv_len || j0 < lo) {
        const uint32_t v0 = kv_smem + stage * kStageBytes + kKeys;
        for (int idx = tid_g; idx < TK * (D / 8); idx += 128) {
          const int r = idx / (D / 8), ch = idx % (D / 8);
          if (j0 + r >= kv_len || j0 + r < lo) {
            const uint32_t addr = v0 + (uint32_t)(r / RPC) * kVPage + (uint32_t)(ch >> 3) * (RPC * 128) + (uint32_t)(r % RPC) * 128 +
                                  (uint32_t)(((ch & 7) ^ (r & 7)) << 4);
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(addr), "r"(0u) : "memory");
          }
        }
      }
      // the row of P: 64 bfloat16 = 128 bytes = eight 16-byte chunks, swizzled by the row
      const uint32_t p_row = p_smem + g * kPBytes + (uint32_t)row * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};\n" ::"r"(p_row + (uint32_t)((ch ^ (row & 7)) << 4)), "r"(packed[4 * ch]),
                     "r"(packed[4 * ch + 1]), "r"(packed[4 * ch + 2]), "r"(packed[4 * ch + 3])
                     : "memory");
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // the stores are visible to the tensor cores' reads
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(g, j & 1));
    }
    // epilogue: O / l
    if (ok && my_tiles > 0) {
      ok = mbar_wait_limited(pv_done(g, (my_tiles - 1) & 1), (uint32_t)((my_tiles - 1) >> 1) & 1u, abortp, 8, &g_attention_tc_error);
    }
    if (ok && my_tiles > 0) {
      tcgen05_fence_after();
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      __nv_bfloat16* dst = valid ? out + ((size_t)(q_start + pr / group) * q_heads + kvh * group + pr % group) * D : nullptr;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tcgen05_ld_32x32b_x32(tmem_o(g) + lane_addr + c * 32, v);
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 ob = __floats2bfloat162_rn(__uint_as_float(v[i + 2 * e]) * inv, __uint_as_float(v[i + 2 * e + 1]) * inv);
              o[e] = *reinterpret_cast<uint32_t*>(&ob);
            }
            *reinterpret_cast<uint4*>(dst + c * 32 + i) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      }
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
  constexpr size_t smem = (size_t)NG * kTcRows * D * 2 + (size_t)tc_stages<D, NG>() * 2 * kTcKeys * D * 2 + (size_t)NG * kTcRows * 128 + 1024;
  auto kernel = attention_prefill_tc_kernel<D, RPC, NG>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attr_set = true;
  }
  launch_kernel(kernel, dim3(items, kv_heads), dim3(64 + NG * 128), smem, s, mq, mk, mv, (__nv_bfloat16*)out, q_indptr, kv_lens, kv_indptr,
                kv_indices, (const int2*)work, q_heads, kv_heads, page_size, scale * kLog2eTc, window);
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
