// Causal grouped-query attention over the paged cache on the tensor cores, for bfloat16.
//
// Definition: src/Starlings.Roost.Ops/CpuOps.cs:181-298 (what attention_generic.cu computes in 32-bit). Scores, the
// running maximum, the exponentials, their sums and the weighted sum of values are kept in 32-bit; the softmax
// weights are rounded to bfloat16 only as the operand of the second product, as the reference's device kernel does
// (kernels/README.md:234-236).
//
// The query heads that share a key/value head are packed into the rows of one tile: packed row r of a request's
// step is (token r / G, head r % G), so a decode step of one token still fills G rows of a 16-row MMA tile and a
// key is loaded once for all G heads. Two kernels share the per-tile arithmetic:
//   * prefill: a CTA of 4 warps owns 64 or 128 packed rows of one request and one key/value head and walks the keys
//     in tiles of 64, double-buffered with cp.async, all warps sharing each tile; with 128 rows a warp carries two row
//     tiles of 16, so each key and value fragment it loads feeds two products;
//   * decode (rows with at most 16 packed rows): a CTA owns one fixed-size chunk of a request's keys; its warps take
//     the chunk's 16-key tiles in turn, each with a three-stage buffer of its own, and merge their partial results in
//     shared memory; a request with several chunks writes (max, sum, unnormalised output) per chunk to a workspace
//     that the merge kernel reduces in chunk order. The chunk size is fixed by the caller, so the order of every sum
//     depends on the request's own length only, never on what else is in the batch.
// Keys outside a request's visible range are never read: their shared-memory rows are zero-filled.
#include "tma.cuh"

namespace roost {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kDecodeTileKeys = 16;  // keys per tile of a decode warp
constexpr int kDecodeStages = 3;     // tiles a decode warp keeps in shared memory

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // src-size 0: the 16 bytes are zero-filled and src is not read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Shared-memory tiles hold rows of D bfloat16 as 16-byte chunks, the chunk index xor-ed with the row so that the
// eight rows an ldmatrix reads fall in different banks.
template <int D>
struct Tile {
  static constexpr int kChunks = D / 8;
  static constexpr int kSwizzle = kChunks >= 8 ? 7 : kChunks - 1;
  __device__ static __forceinline__ uint32_t offset(int row, int chunk) { return (uint32_t)(row * kChunks + (chunk ^ (row & kSwizzle))) * 16u; }
};

// Loads keys [j0, j0 + ROWS) of one key/value head into a K and a V tile. Keys outside [lo, hi] are zero-filled.
// A thread owns one 16-byte chunk column and every (NTHREADS / chunks)-th row. The block-table lookups of all its
// rows are issued first, then the copies, so the lookups' latencies overlap instead of adding up in front of each copy.
template <int D, int ROWS, int NTHREADS>
__device__ __forceinline__ void load_kv_tile(uint32_t k_smem, uint32_t v_smem, const __nv_bfloat16* __restrict__ k_pool,
                                             const __nv_bfloat16* __restrict__ v_pool, const int32_t* __restrict__ pages,
                                             int page_size, int page_shift, int kv_heads, int kvh, int j0, int lo, int hi, int tid) {
  constexpr int C = Tile<D>::kChunks;
  static_assert(NTHREADS % C == 0 && NTHREADS >= C, "a row's chunks must divide the threads");
  constexpr int ROWS_PER_PASS = NTHREADS / C;
  constexpr int ITER = (ROWS + ROWS_PER_PASS - 1) / ROWS_PER_PASS;
  const int ch = tid % C;
  const int r0 = tid / C;
  int page[ITER];
#pragma unroll
  for (int k = 0; k < ITER; ++k) {
    const int j = j0 + r0 + k * ROWS_PER_PASS;
    const bool valid = j >= lo && j <= hi && (r0 + k * ROWS_PER_PASS) < ROWS;
    page[k] = valid ? pages[page_shift >= 0 ? (j >> page_shift) : (j / page_size)] : -1;
  }
#pragma unroll
  for (int k = 0; k < ITER; ++k) {
    const int r = r0 + k * ROWS_PER_PASS;
    if (r < ROWS) {
      const int j = j0 + r;
      const bool valid = page[k] >= 0;
      const int off = page_shift >= 0 ? (j & (page_size - 1)) : (j % page_size);
      const size_t base = valid ? (((size_t)page[k] * kv_heads + kvh) * page_size + off) * D + ch * 8 : 0;
      cp_async_16(k_smem + Tile<D>::offset(r, ch), k_pool + base, valid);
      cp_async_16(v_smem + Tile<D>::offset(r, ch), v_pool + base, valid);
    }
  }
}

// The state of one warp's 16 packed rows: thread t holds rows t/4 and t/4 + 8.
template <int D>
struct RowState {
  float o[D / 8][4];
  float m[2];  // running maximum of the scaled scores (in log2 units)
  float l[2];  // running sum of 2^(s - m)
};

// One warp, 16 query rows, BN keys from a K/V tile laid out as L: S = Q K^T, online softmax, O += P V. q_frag(kk, a0..a3)
// yields the A operand of k-step kk. qpos/qlo: per held row, the last and first visible key position (qlo > qpos masks
// the row).
template <int D, int BN, typename L, typename QFrag>
__device__ __forceinline__ void attend_core(RowState<D>& st, QFrag q_frag, uint32_t k_smem, uint32_t v_smem, int j0, const int (&qpos)[2],
                                            const int (&qlo)[2], float scale_log2, int lane) {
  constexpr int NT = BN / 8;
  float s[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a0, a1, a2, a3;
    q_frag(kk, a0, a1, a2, a3);
#pragma unroll
    for (int n2 = 0; n2 < NT / 2; ++n2) {
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(k_smem + L::offset(n2 * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
      mma_bf16(s[2 * n2], a0, a1, a2, a3, b0, b1);
      mma_bf16(s[2 * n2 + 1], a0, a1, a2, a3, b2, b3);
    }
  }
  // mask and running maximum; a tile every key of which both rows see needs no per-element test
  float mx[2] = {-INFINITY, -INFINITY};
  const bool all_visible = j0 + BN - 1 <= min(qpos[0], qpos[1]) && j0 >= max(qlo[0], qlo[1]);
  if (__all_sync(0xffffffffu, all_visible)) {
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s[n][e] *= scale_log2;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
      }
    }
  } else {
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const int j = j0 + n * 8 + (lane & 3) * 2 + (e & 1);
        const float v = (j <= qpos[r] && j >= qlo[r]) ? s[n][e] * scale_log2 : -INFINITY;
        s[n][e] = v;
        mx[r] = fmaxf(mx[r], v);
      }
    }
  }
  float corr[2], msafe[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float m_new = fmaxf(st.m[r], mx[r]);
    msafe[r] = m_new == -INFINITY ? 0.f : m_new;  // a row that has seen no key yet: every weight below is 0
    corr[r] = exp2f(st.m[r] - msafe[r]);          // 0 when st.m is -inf
    st.m[r] = m_new;
  }
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int n = 0; n < NT; ++n) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float p = exp2f(s[n][e] - msafe[e >> 1]);
      s[n][e] = p;
      sum[e >> 1] += p;
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
    sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
    st.l[r] = st.l[r] * corr[r] + sum[r];
  }
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    st.o[n][0] *= corr[0];
    st.o[n][1] *= corr[0];
    st.o[n][2] *= corr[1];
    st.o[n][3] *= corr[1];
  }
  // O += P V
#pragma unroll
  for (int kk = 0; kk < BN / 16; ++kk) {
    const uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    const uint32_t a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    const uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    const uint32_t a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int n2 = 0; n2 < D / 16; ++n2) {
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(v_smem + L::offset(kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), n2 * 2 + (lane >> 4)), b0, b1, b2, b3);
      mma_bf16(st.o[2 * n2], a0, a1, a2, a3, b0, b1);
      mma_bf16(st.o[2 * n2 + 1], a0, a1, a2, a3, b2, b3);
    }
  }
}

// The same with the query rows q_row0..+15 of a shared-memory tile as the A operand and K/V tiles in the same layout.
template <int D, int BN>
__device__ __forceinline__ void attend_tile(RowState<D>& st, uint32_t q_smem, int q_row0, uint32_t k_smem, uint32_t v_smem, int j0,
                                            const int (&qpos)[2], const int (&qlo)[2], float scale_log2, int lane) {
  attend_core<D, BN, Tile<D>>(
      st,
      [&](int kk, uint32_t& a0, uint32_t& a1, uint32_t& a2, uint32_t& a3) {
        ldmatrix_x4(q_smem + Tile<D>::offset(q_row0 + (lane & 15), kk * 2 + (lane >> 4)), a0, a1, a2, a3);
      },
      k_smem, v_smem, j0, qpos, qlo, scale_log2, lane);
}

// The same for MT row tiles of 16 per warp: a key or value fragment loaded from shared memory feeds MT products, which is
// what lifts the ratio of tensor-core work to shared-memory traffic in prefill. Keys key_row0 .. key_row0 + BN - 1 of the
// K/V tile are used; j0 is the position of the first of them.
template <int D, int MT>
struct RowStateM {
  float o[MT][D / 8][4];
  float m[MT][2];
  float l[MT][2];
};

template <int D, int BN, int MT>
__device__ __forceinline__ void attend_tile_m(RowStateM<D, MT>& st, uint32_t q_smem, int q_row0, uint32_t k_smem, uint32_t v_smem,
                                              int key_row0, int j0, const int (&qpos)[MT][2], const int (&qlo)[MT][2], float scale_log2,
                                              int lane) {
  constexpr int NT = BN / 8;
  float s[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int n = 0; n < NT; ++n) s[mt][n][0] = s[mt][n][1] = s[mt][n][2] = s[mt][n][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
      ldmatrix_x4(q_smem + Tile<D>::offset(q_row0 + mt * 16 + (lane & 15), kk * 2 + (lane >> 4)), a[mt][0], a[mt][1], a[mt][2], a[mt][3]);
#pragma unroll
    for (int n2 = 0; n2 < NT / 2; ++n2) {
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(k_smem + Tile<D>::offset(key_row0 + n2 * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        mma_bf16(s[mt][2 * n2], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b0, b1);
        mma_bf16(s[mt][2 * n2 + 1], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b2, b3);
      }
    }
  }
  float corr[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    float mx[2] = {-INFINITY, -INFINITY};
    const bool all_visible = j0 + BN - 1 <= min(qpos[mt][0], qpos[mt][1]) && j0 >= max(qlo[mt][0], qlo[mt][1]);
    if (__all_sync(0xffffffffu, all_visible)) {
#pragma unroll
      for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[mt][n][e] *= scale_log2;
          mx[e >> 1] = fmaxf(mx[e >> 1], s[mt][n][e]);
        }
      }
    } else {
#pragma unroll
      for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          const int j = j0 + n * 8 + (lane & 3) * 2 + (e & 1);
          const float v = (j <= qpos[mt][r] && j >= qlo[mt][r]) ? s[mt][n][e] * scale_log2 : -INFINITY;
          s[mt][n][e] = v;
          mx[r] = fmaxf(mx[r], v);
        }
      }
    }
    float msafe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(st.m[mt][r], mx[r]);
      msafe[r] = m_new == -INFINITY ? 0.f : m_new;
      corr[mt][r] = exp2f(st.m[mt][r] - msafe[r]);
      st.m[mt][r] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = exp2f(s[mt][n][e] - msafe[e >> 1]);
        s[mt][n][e] = p;
        sum[e >> 1] += p;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
      sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
      st.l[mt][r] = st.l[mt][r] * corr[mt][r] + sum[r];
    }
    // the running maximum rarely moves after a row's first tiles: a factor of exactly 1 for every row of the warp needs
    // no pass over the accumulator
    if (__any_sync(0xffffffffu, corr[mt][0] != 1.0f || corr[mt][1] != 1.0f)) {
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        st.o[mt][n][0] *= corr[mt][0];
        st.o[mt][n][1] *= corr[mt][0];
        st.o[mt][n][2] *= corr[mt][1];
        st.o[mt][n][3] *= corr[mt][1];
      }
    }
  }
#pragma unroll
  for (int kk = 0; kk < BN / 16; ++kk) {
    uint32_t a[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      a[mt][0] = pack_bf16(s[mt][2 * kk][0], s[mt][2 * kk][1]);
      a[mt][1] = pack_bf16(s[mt][2 * kk][2], s[mt][2 * kk][3]);
      a[mt][2] = pack_bf16(s[mt][2 * kk + 1][0], s[mt][2 * kk + 1][1]);
      a[mt][3] = pack_bf16(s[mt][2 * kk + 1][2], s[mt][2 * kk + 1][3]);
    }
#pragma unroll
    for (int n2 = 0; n2 < D / 16; ++n2) {
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(v_smem + Tile<D>::offset(key_row0 + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), n2 * 2 + (lane >> 4)), b0, b1, b2, b3);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        mma_bf16(st.o[mt][2 * n2], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b0, b1);
        mma_bf16(st.o[mt][2 * n2 + 1], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b2, b3);
      }
    }
  }
}


// Loads packed query rows [row0, row0 + ROWS) of one request and key/value head into a Q tile (rows past the
// request's last packed row are zero-filled).
template <int D, int ROWS, int NTHREADS>
__device__ __forceinline__ void load_q_tile(uint32_t q_smem, const __nv_bfloat16* __restrict__ q, int q_start, int q_heads, int group,
                                            int kvh, int row0, int rows_total, int tid) {
  constexpr int C = Tile<D>::kChunks;
  for (int i = tid; i < ROWS * C; i += NTHREADS) {
    const int r = i / C, ch = i % C;
    const int pr = row0 + r;
    const bool valid = pr < rows_total;
    size_t src = 0;
    if (valid) src = ((size_t)(q_start + pr / group) * q_heads + kvh * group + pr % group) * D + ch * 8;
    cp_async_16(q_smem + Tile<D>::offset(r, ch), q + src, valid);
  }
}

// ------------------------------------------------------------------------------------------------ prefill
// work[i] = (batch row, first packed row of the tile); a tile is 64 * MT packed rows, 16 * MT per warp
template <int D, int MT>
__global__ void __launch_bounds__(128) attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                                                                const __nv_bfloat16* __restrict__ k_pool,
                                                                const __nv_bfloat16* __restrict__ v_pool,
                                                                const int32_t* __restrict__ q_indptr, const int32_t* __restrict__ kv_lens,
                                                                const int32_t* __restrict__ kv_indptr,
                                                                const int32_t* __restrict__ kv_indices, const int2* __restrict__ work,
                                                                int q_heads, int kv_heads, int page_size, int page_shift, float scale_log2, int window) {
  constexpr int BM = 64 * MT, BN = 64, HALF = 32, NT = 128;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const uint32_t smem = (uint32_t)__cvta_generic_to_shared(smem_raw);
  constexpr uint32_t kTileBytes = BN * D * 2;
  const uint32_t q_smem = smem;
  const uint32_t k_smem[2] = {smem + BM * D * 2, smem + BM * D * 2 + 2 * kTileBytes};
  const uint32_t v_smem[2] = {k_smem[0] + kTileBytes, k_smem[1] + kTileBytes};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_launch_dependents();
  pdl_wait();
  const int2 w = work[blockIdx.x];
  const int b = w.x, row0 = w.y;
  if (b < 0) return;  // padding of a fixed-size work list
  const int kvh = blockIdx.y;
  const int group = q_heads / kv_heads;
  const int q_start = q_indptr[b];
  const int n = q_indptr[b + 1] - q_start;
  const int kv_len = kv_lens[b];
  const int pos0 = kv_len - n;
  const int rows_total = n * group;
  const int32_t* pages = kv_indices + kv_indptr[b];

  // this thread's rows: two in each of the warp's MT row tiles
  int qpos[MT][2], qlo[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int pr = row0 + warp * 16 * MT + mt * 16 + (lane >> 2) + r * 8;
      if (pr < rows_total) {
        qpos[mt][r] = pos0 + pr / group;
        qlo[mt][r] = window > 0 ? max(0, qpos[mt][r] - window + 1) : 0;
      } else {
        qpos[mt][r] = -1;  // sees nothing
        qlo[mt][r] = 0;
      }
    }
  }
  // the tile's key range, and this warp's own (a warp skips key tiles none of its rows can see)
  const int last_row = min(row0 + BM, rows_total) - 1;
  const int hi = pos0 + last_row / group;
  const int lo = window > 0 ? max(0, pos0 + row0 / group - window + 1) : 0;
  const int t0 = lo / BN, t1 = hi / BN;
  const int warp_first = row0 + warp * 16 * MT;
  const int warp_last = min(warp_first + 16 * MT, rows_total) - 1;
  const int warp_hi = warp_last >= warp_first ? pos0 + warp_last / group : -1;
  const int warp_lo = window > 0 ? max(0, pos0 + warp_first / group - window + 1) : 0;

  load_q_tile<D, BM, NT>(q_smem, q, q_start, q_heads, group, kvh, row0, rows_total, tid);
  load_kv_tile<D, BN, NT>(k_smem[0], v_smem[0], k_pool, v_pool, pages, page_size, page_shift, kv_heads, kvh, t0 * BN, lo, hi, tid);
  cp_async_commit();

  RowStateM<D, MT> st;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int i = 0; i < D / 8; ++i) st.o[mt][i][0] = st.o[mt][i][1] = st.o[mt][i][2] = st.o[mt][i][3] = 0.f;
    st.m[mt][0] = st.m[mt][1] = -INFINITY;
    st.l[mt][0] = st.l[mt][1] = 0.f;
  }

  for (int t = t0; t <= t1; ++t) {
    const int stage = (t - t0) & 1;
    if (t + 1 <= t1) {
      load_kv_tile<D, BN, NT>(k_smem[stage ^ 1], v_smem[stage ^ 1], k_pool, v_pool, pages, page_size, page_shift, kv_heads, kvh, (t + 1) * BN, lo, hi, tid);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
#pragma unroll
    for (int half = 0; half < BN / HALF; ++half) {
      const int j0 = t * BN + half * HALF;
      if (j0 <= warp_hi && j0 + HALF - 1 >= warp_lo) {  // uniform in the warp
        attend_tile_m<D, HALF, MT>(st, q_smem, warp * 16 * MT, k_smem[stage], v_smem[stage], half * HALF, j0, qpos, qlo, scale_log2, lane);
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int pr = row0 + warp * 16 * MT + mt * 16 + (lane >> 2) + r * 8;
      if (pr >= rows_total) continue;
      const float inv = st.l[mt][r] > 0.f ? 1.0f / st.l[mt][r] : 0.f;
      __nv_bfloat16* dst = out + ((size_t)(q_start + pr / group) * q_heads + kvh * group + pr % group) * D + (lane & 3) * 2;
#pragma unroll
      for (int nn = 0; nn < D / 8; ++nn) {
        *reinterpret_cast<uint32_t*>(dst + nn * 8) = pack_bf16(st.o[mt][nn][2 * r] * inv, st.o[mt][nn][2 * r + 1] * inv);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ decode
// work[i] = (batch row, first key of the chunk, one past its last key, partial slot or -1 for a row with one chunk)
// Partial results of slot s and key/value head h: part_o[(s * kv_heads + h) * 16 + row][D], part_ml[...][2].
// slot_limit: partial slots the workspace holds. An item that names a slot at or beyond it is skipped and code 9 is
// recorded for roost_attention_status(): a work list that does not match the workspace must not write past it.
__device__ int g_attention_error = 0;   // 0, or the code of the first fault a decode kernel met since it was last read
constexpr int kNoSlotLimit = 0x7fffffff;
template <int D, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32)
    attention_decode_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ k_pool,
                            const __nv_bfloat16* __restrict__ v_pool, const int32_t* __restrict__ q_indptr,
                            const int32_t* __restrict__ kv_lens, const int32_t* __restrict__ kv_indptr,
                            const int32_t* __restrict__ kv_indices, const int4* __restrict__ work, float* __restrict__ part_o,
                            float* __restrict__ part_ml, int q_heads, int kv_heads, int page_size, int page_shift, float scale_log2, int window,
                            int slot_limit) {
  constexpr int BN = kDecodeTileKeys, STAGES = kDecodeStages;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const uint32_t smem = (uint32_t)__cvta_generic_to_shared(smem_raw);
  constexpr uint32_t kTileBytes = BN * D * 2;
  constexpr uint32_t kQBytes = 16 * D * 2;
  constexpr uint32_t kStageBytes = 2 * kTileBytes;             // K then V
  constexpr uint32_t kWarpBytes = STAGES * kStageBytes;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t q_smem = smem;
  const uint32_t wbase = smem + kQBytes + warp * kWarpBytes;

  pdl_launch_dependents(4);
  pdl_wait(4);
  const int4 w = work[blockIdx.x];
  const int b = w.x, kv_begin = w.y, kv_end = w.z, slot = w.w;
  if (b < 0) return;  // padding of a fixed-size work list
  if (slot >= slot_limit) {
    if (tid == 0) atomicCAS(&g_attention_error, 0, 9);
    return;
  }
  const int kvh = blockIdx.y;
  const int group = q_heads / kv_heads;
  const int q_start = q_indptr[b];
  const int n = q_indptr[b + 1] - q_start;
  const int kv_len = kv_lens[b];
  const int pos0 = kv_len - n;
  const int rows_total = n * group;  // at most 16
  const int32_t* pages = kv_indices + kv_indptr[b];

  int qpos[2], qlo[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int pr = (lane >> 2) + r * 8;
    if (pr < rows_total) {
      qpos[r] = pos0 + pr / group;
      qlo[r] = window > 0 ? max(0, qpos[r] - window + 1) : 0;
    } else {
      qpos[r] = -1;
      qlo[r] = 0;
    }
  }
  // keys this chunk may read: inside the chunk, not beyond the last query, not before the first query's window
  const int hi = min(kv_end - 1, kv_len - 1);
  const int lo = max(kv_begin, window > 0 ? max(0, pos0 - window + 1) : 0);

  load_q_tile<D, 16, NWARPS * 32>(q_smem, q, q_start, q_heads, group, kvh, 0, rows_total, tid);
  cp_async_commit();

  RowState<D> st;
#pragma unroll
  for (int i = 0; i < D / 8; ++i) st.o[i][0] = st.o[i][1] = st.o[i][2] = st.o[i][3] = 0.f;
  st.m[0] = st.m[1] = -INFINITY;
  st.l[0] = st.l[1] = 0.f;

  // tiles of the chunk from the first visible key on, taken by the warps in turn; each warp keeps STAGES - 1 tiles in
  // flight ahead of the one it computes on. One commit group per tile slot, empty when the warp has no such tile, so
  // that the group count is the same for every lane and iteration.
  const int t0 = lo / BN;
  const int ntiles = hi >= lo ? (hi / BN - t0 + 1) : 0;
  const int mine = warp < ntiles ? (ntiles - warp + NWARPS - 1) / NWARPS : 0;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < mine) {
      const uint32_t dst = wbase + s * kStageBytes;
      load_kv_tile<D, BN, 32>(dst, dst + kTileBytes, k_pool, v_pool, pages, page_size, page_shift, kv_heads, kvh, (t0 + warp + s * NWARPS) * BN, lo, hi, lane);
    }
    cp_async_commit();
  }
  cp_async_wait<STAGES - 1>();  // the Q tile (the oldest group); made visible to all by the barrier
  __syncthreads();
  for (int i = 0; i < mine; ++i) {
    const int t = t0 + warp + i * NWARPS;
    const uint32_t cur = wbase + (i % STAGES) * kStageBytes;
    if (i + STAGES - 1 < mine) {
      const uint32_t dst = wbase + ((i + STAGES - 1) % STAGES) * kStageBytes;
      load_kv_tile<D, BN, 32>(dst, dst + kTileBytes, k_pool, v_pool, pages, page_size, page_shift, kv_heads, kvh, (t + (STAGES - 1) * NWARPS) * BN, lo, hi, lane);
    }
    cp_async_commit();
    cp_async_wait<STAGES - 1>();  // all but the newest STAGES - 1 groups are done: tile i has arrived
    __syncwarp();
    attend_tile<D, BN>(st, q_smem, 0, cur, cur + kTileBytes, t * BN, qpos, qlo, scale_log2, lane);
    __syncwarp();  // every lane is done with `cur` before a later iteration loads into it
  }
  cp_async_wait<0>();
  __syncthreads();

  // merge the warps' states through shared memory (in warp order), then write the chunk's result
  float* sm_o = reinterpret_cast<float*>(smem_raw + kQBytes);          // [NWARPS][16][D]
  float* sm_ml = sm_o + NWARPS * 16 * D;                               // [NWARPS][16][2]
  static_assert(NWARPS * 16 * D * 4 + NWARPS * 16 * 2 * 4 <= NWARPS * kWarpBytes, "merge scratch does not fit in the tile buffers");
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = (lane >> 2) + r * 8;
    if (row < rows_total) {
      float* dst = sm_o + ((size_t)warp * 16 + row) * D + (lane & 3) * 2;
#pragma unroll
      for (int nn = 0; nn < D / 8; ++nn) {
        dst[nn * 8] = st.o[nn][2 * r];
        dst[nn * 8 + 1] = st.o[nn][2 * r + 1];
      }
      if ((lane & 3) == 0) {
        sm_ml[(warp * 16 + row) * 2] = st.m[r];
        sm_ml[(warp * 16 + row) * 2 + 1] = st.l[r];
      }
    }
  }
  __syncthreads();
  for (int idx = tid; idx < rows_total * D; idx += NWARPS * 32) {
    const int row = idx / D, col = idx % D;
    float m = -INFINITY;
#pragma unroll
    for (int ww = 0; ww < NWARPS; ++ww) m = fmaxf(m, sm_ml[(ww * 16 + row) * 2]);
    const float msafe = m == -INFINITY ? 0.f : m;
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int ww = 0; ww < NWARPS; ++ww) {
      const float f = exp2f(sm_ml[(ww * 16 + row) * 2] - msafe);
      l += sm_ml[(ww * 16 + row) * 2 + 1] * f;
      o += sm_o[((size_t)ww * 16 + row) * D + col] * f;
    }
    if (slot < 0) {
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      out[((size_t)(q_start + row / group) * q_heads + kvh * group + row % group) * D + col] = __float2bfloat16_rn(o * inv);
    } else {
      const size_t pr = ((size_t)slot * kv_heads + kvh) * 16 + row;
      part_o[pr * D + col] = o;
      if (col == 0) {
        part_ml[pr * 2] = m;
        part_ml[pr * 2 + 1] = l;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ decode, keys and values by TMA
// The same chunks, streamed by the copy engine through one ring of shared-memory stages per CTA. The CTAs are persistent:
// CTA c takes the (chunk, key/value head) pairs c, c + G, c + 2G, ... of the work list, and the ring keeps running
// across them, so the loads of the next chunk are in flight while the last tiles of this one are computed and merged.
//   warp 4 (producer): per chunk it reads the chunk's row of the step tables (one chunk ahead, in three dependent rounds
//     spread over the tiles of the chunk before, so that their latencies are hidden), copies the chunk's Q tile into a
//     two-entry ring and publishes the chunk's facts beside it (the descriptor's barrier completes when both are in
//     shared memory), and walks the chunk in tiles of 32 keys: it looks the pages up (32 block-table entries a load,
//     kept one a lane as pool rows), waits for a free stage and issues one tensor copy per page that brings the page's
//     keys and values (a 4-D box over the pool: 64 columns x rows x column blocks x {K, V}) into 128-byte-swizzled
//     shared memory; the copies complete on the stage's barrier.
//   warps 0..3 (consumers): tile g of the CTA's stream goes to warp g % 4. Each takes the query fragments into registers
//     when a chunk begins, keeps a running state of its own, hands the stage back after its products, and the four
//     merge through shared memory in warp order when the chunk ends, two packed rows a pass.
// A page is copied whole: rows of a tile that lie outside the row's visible keys hold whatever the pool holds there.
// Their scores are masked by position; their value rows are zeroed in shared memory by the consuming warp before the
// second product (only the first and last tile of a chunk have such rows), so nothing outside the visible range reaches
// a result. A page the request has given back (block-table entry -1) is replaced by the request's last page.
// Every wait is bounded: a wait given up raises the CTA's abort flag, records a code that roost_attention_status()
// returns, and the CTA lets its copies land before it exits.
constexpr int kTmaTileKeys = 32;
constexpr int kTmaConsumers = 4;
constexpr int kTmaMergeRows = 2;  // packed rows merged per pass
constexpr int kEarlyTiles = 2;    // tiles of a CTA's first chunk whose copies are issued before the wait for the kernel in front

// A tile of TK keys as the copies leave it: [page of RPC rows][K, V][D / 64 column blocks][RPC][64 bfloat16], 128-byte
// swizzle, 1024-byte aligned. offset() is relative to the tile's keys; the values follow at kValues.
template <int D, int RPC>
struct TileTma {
  static constexpr uint32_t kValues = (D / 64) * RPC * 128;
  static constexpr uint32_t kPage = 2 * kValues;
  __device__ static __forceinline__ uint32_t offset(int row, int chunk) {
    return (uint32_t)((row / RPC) * kPage + (chunk >> 3) * RPC * 128 + (row % RPC) * 128 + (((chunk & 7) ^ (row & 7)) << 4));
  }
};

struct DecodeChunk {  // what the producer tells the consumers about a chunk
  int b, kvh, slot, q_start, n, kv_len, lo, hi, t0, ntiles;
};

__device__ __forceinline__ uint32_t decode_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
// Every thread of the cluster that has not exited arrives and waits (the producer warps have left by then, or leave
// soon: a thread that exits no longer counts).
__device__ __forceinline__ void decode_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release;\nbarrier.cluster.wait.acquire;\n" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote));
  return v;
}

template <int D>
constexpr int tma_decode_stages() {
  return (96 * 1024) / (2 * kTmaTileKeys * D * 2);  // 6 at head size 128, 12 at 64
}

template <int D, int RPC>
__global__ void __launch_bounds__((kTmaConsumers + 1) * 32, 2)
    attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_kv, const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                                const int32_t* __restrict__ q_indptr, const int32_t* __restrict__ kv_lens,
                                const int32_t* __restrict__ kv_indptr, const int32_t* __restrict__ kv_indices,
                                const int4* __restrict__ work, int items, float* __restrict__ part_o, float* __restrict__ part_ml, int q_heads,
                                int kv_heads, int page_size, float scale_log2, int window, int cluster_chunks) {
  // cluster_chunks = S > 0: the grid is clusters of S CTAs, one cluster a (row, key/value head), the row's work items S in
  // a row of the list (some of them empty); CTA r of a cluster takes the r-th, leaves its result in its own shared memory
  // and the CTAs combine the S results in chunk order, with the merge kernel's arithmetic, through distributed shared
  // memory (each a share of the row's values): no partial results in global memory and no merge kernel.
  constexpr int TK = kTmaTileKeys, STAGES = tma_decode_stages<D>(), NW = kTmaConsumers, MR = kTmaMergeRows;
  constexpr uint32_t kStageBytes = 2 * TK * D * 2;  // keys and values of TK positions
  constexpr uint32_t kQBytes = 16 * D * 2;
  constexpr int kScratchStride = D + 8;              // floats; the pad spreads the rows over the banks
  using L = TileTma<D, RPC>;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = ((uint32_t)__cvta_generic_to_shared(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem_gen = smem_raw + (smem_base - (uint32_t)__cvta_generic_to_shared(smem_raw));
  const uint32_t q_smem = smem_base + STAGES * kStageBytes;
  float* sm_o = reinterpret_cast<float*>(smem_gen + STAGES * kStageBytes + 2 * kQBytes);  // [NW][MR][kScratchStride]
  float* sm_ml = sm_o + NW * MR * kScratchStride;                                      // [NW][MR][2]
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
  __shared__ DecodeChunk desc[2];
  __shared__ int abort_flag;
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(bars);
  auto full_bar = [&](int st) { return bar0 + 8u * st; };
  auto empty_bar = [&](int st) { return bar0 + 8u * (STAGES + st); };
  auto desc_full = [&](int d) { return bar0 + 8u * (2 * STAGES + d); };
  auto desc_empty = [&](int d) { return bar0 + 8u * (2 * STAGES + 2 + d); };
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    prefetch_tensormap(&map_kv);
    abort_flag = 0;
    for (int st = 0; st < STAGES; ++st) {
      mbar_init(full_bar(st), 1);
      mbar_init(empty_bar(st), 1);
    }
    for (int d = 0; d < 2; ++d) {
      mbar_init(desc_full(d), 33);  // the producer's 32 copy completions and its descriptor
      mbar_init(desc_empty(d), NW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  pdl_launch_dependents(4);
  __syncthreads();  // the barriers are initialised
  const int group = q_heads / kv_heads;
  const long long total = (long long)items * kv_heads;
  volatile int* abortp = &abort_flag;
  // What the kernel before this one on the stream writes (the step's queries, and the keys and values of the step's own
  // tokens) is first touched after pdl_wait(). The step's tables were copied to the device before the step's first
  // kernel, and pages that hold only earlier tokens were written by earlier steps: the producer reads the first and
  // starts copying the second while the kernel before is still running.

  if (warp == NW) {
    // ---- producer: all lanes walk the loops (a lane holds one block-table entry of the current 32, as the pool row its
    // page starts at); lane 0 waits, publishes and issues. What the next chunk needs from the step tables is fetched in
    // three dependent rounds (work item; the row's lengths; its block-table entries) spread over the tiles of this one.
    constexpr int COPIES = TK / RPC;
    const int page_shift = 31 - __clz(page_size);  // a power of two here
    bool ok = true;
    int g = 0;  // tiles issued so far
    // the chunk being fetched: work item (first fetch), row facts (second), chunk and block-table entries (third)
    long long nf = blockIdx.x;
    int4 nw = make_int4(-1, 0, 0, 0);
    int nq0 = 0, nq1 = 0, nkvl = 0, ntbl = 0;
    DecodeChunk nc;
    int n_fallback = 0, n_cur = -1, n_nxt = -1;
    auto item_of = [&](long long f) -> long long {
      if (cluster_chunks > 0) {  // fewer than 2^31 items x heads here
        const unsigned u = (unsigned)f, pair = u / (unsigned)cluster_chunks;
        return (long long)((pair / (unsigned)kv_heads) * (unsigned)cluster_chunks + u % (unsigned)cluster_chunks);
      }
      return f / kv_heads;
    };
    auto round1 = [&]() { nw = nf < total ? work[item_of(nf)] : make_int4(-1, 0, 0, 0); };
    auto round2 = [&]() {
      if (nw.x >= 0) {
        nq0 = q_indptr[nw.x];
        nq1 = q_indptr[nw.x + 1];
        nkvl = kv_lens[nw.x];
        ntbl = kv_indptr[nw.x];
      }
    };
    auto round3 = [&]() {
      nc.b = nw.x;  // padding entries (batch row -1) end the list
      nc.ntiles = 0;
      if (nc.b >= 0) {
        nc.kvh = cluster_chunks > 0 ? (int)(((unsigned)nf / (unsigned)cluster_chunks) % (unsigned)kv_heads) : (int)(nf % kv_heads);
        nc.slot = nw.w;
        nc.q_start = nq0;
        nc.n = nq1 - nq0;
        nc.kv_len = nkvl;
        const int pos0 = nc.kv_len - nc.n;
        nc.hi = min(nw.z - 1, nc.kv_len - 1);
        nc.lo = max(nw.y, window > 0 ? max(0, pos0 - window + 1) : 0);
        nc.t0 = nc.lo / TK;
        nc.ntiles = nc.hi >= nc.lo ? (nc.hi / TK - nc.t0 + 1) : 0;
        if (nc.ntiles > 0) {
          const int32_t* pages = kv_indices + ntbl;
          const int p_first = (nc.t0 * TK) >> page_shift, p_last = nc.hi >> page_shift;
          n_fallback = pages[p_last];
          n_cur = p_first + lane <= p_last ? pages[p_first + lane] : -1;
          n_nxt = p_first + 32 + lane <= p_last ? pages[p_first + 32 + lane] : -1;
        }
      }
    };
#ifdef ROOST_TRACE
    unsigned long long trp[7] = {trace_now(), 0, 0, 0, 0, 0, 0};
#endif
    round1();
    round2();
    round3();
#ifdef ROOST_TRACE
    trp[1] = trace_now();   // the first chunk's tables are known
#endif
    for (int k = 0; ok; ++k) {
      const DecodeChunk c = nc;
      const int fallback = n_fallback;
      const int first_entry = n_cur;
      int nxt_entry = n_nxt;
      const int32_t* pages = kv_indices + ntbl;
      nf += gridDim.x;
      int rounds = 0;  // rounds of the next chunk's fetch done so far
      if (c.b >= 0) {
        round1();
        rounds = 1;
      }
      const int p_first = (c.t0 * TK) >> page_shift, p_last = c.hi >> page_shift;
      auto row_of = [&](int p, int entry) {  // first pool row of page p of the request, given its block-table entry
        const bool visible = ((p + 1) << page_shift) > c.lo && (p << page_shift) <= c.hi;
        return ((visible && entry >= 0 ? entry : fallback) * kv_heads + c.kvh) << page_shift;
      };
      int batch0 = p_first;  // the page lane 0 holds
      int cur = c.b >= 0 ? row_of(batch0 + lane, first_entry) : 0;
      auto issue = [&](int i) {  // the copies of tile i of the chunk
        if (i == 2 && rounds == 1) {
          round2();
          rounds = 2;
        } else if (i == 5 && rounds == 2) {
          round3();
          rounds = 3;
        }
        const int stage = g % STAGES;
        const uint32_t dst = smem_base + stage * kStageBytes;
        const int j = (c.t0 + i) * TK;
        if ((j >> page_shift) >= batch0 + 32) {  // uniform in the warp
          batch0 += 32;
          cur = row_of(batch0 + lane, nxt_entry);
          nxt_entry = batch0 + 32 + lane <= p_last ? pages[batch0 + 32 + lane] : -1;
        }
        int rows[COPIES];
#pragma unroll
        for (int cc = 0; cc < COPIES; ++cc) {
          const int jc = j + cc * RPC;
          rows[cc] = __shfl_sync(0xffffffffu, cur, ((jc >> page_shift) - batch0) & 31) + (jc & (page_size - 1));
        }
        if (lane == 0) {
          if (g >= STAGES) ok = mbar_wait_limited(empty_bar(stage), (uint32_t)((g / STAGES) - 1) & 1u, abortp, 1, &g_attention_error);
          if (ok) {
            mbar_expect_tx(full_bar(stage), kStageBytes);
#pragma unroll
            for (int cc = 0; cc < COPIES; ++cc) tma_load_4d(dst + cc * L::kPage, &map_kv, full_bar(stage), 0, rows[cc], 0, 0);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        ++g;
      };
      int issued = 0;
      if (k == 0) {
        // the CTA's first chunk, when it lies wholly before the step's own tokens: its first tiles are on their way
        // before the kernel in front has finished
        if (c.b >= 0 && c.hi < c.kv_len - c.n) {
          // (a tile's copies take the issuing lane about 0.3 us, and the consumers cannot begin before the descriptor and Q,
          // which follow the wait: two tiles are as much as fits before the kernel in front is usually done)
          const int early = c.ntiles < kEarlyTiles ? c.ntiles : kEarlyTiles;
          for (; issued < early && ok; ++issued) issue(issued);
        }
#ifdef ROOST_TRACE
        trp[4] = trace_now();   // the early copies are issued
#endif
        pdl_wait(4);
#ifdef ROOST_TRACE
        trp[5] = trace_now();   // the kernel in front has finished
#endif
      }
      if (lane == 0 && k >= 2) ok = mbar_wait_limited(desc_empty(k & 1), (uint32_t)((k >> 1) - 1) & 1u, abortp, 4, &g_attention_error);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      // the chunk's Q tile, then the descriptor: the barrier completes when both are in shared memory
      if (c.b >= 0) load_q_tile<D, 16, 32>(q_smem + (k & 1) * kQBytes, q, c.q_start, q_heads, group, c.kvh, 0, c.n * group, lane);
#ifdef ROOST_TRACE
      if (k == 0) trp[6] = trace_now();   // the copies of Q are issued
#endif
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(desc_full(k & 1)) : "memory");
      if (lane == 0) {
        desc[k & 1] = c;
        mbar_arrive(desc_full(k & 1));  // releases the descriptor to the consumers
      }
      if (c.b < 0) break;
#ifdef ROOST_TRACE
      if (k == 0) trp[2] = trace_now();   // the descriptor and Q are on their way
#endif
      for (int i = issued; i < c.ntiles && ok; ++i) issue(i);
#ifdef ROOST_TRACE
      if (k == 0) trp[3] = trace_now();   // the chunk's last copy is issued
#endif
      if (rounds < 2) round2();
      if (rounds < 3) round3();
    }
#ifdef ROOST_TRACE
    if (lane == 0 && (blockIdx.x & 7) == 0) {
      trace_flush(4 * 4 + 3, blockIdx.x * 16, trp, 4);
      trace_flush(4 * 4 + 3, blockIdx.x * 16 + 10, trp + 4, 3);
    }
#endif
    if (*abortp) {  // copies in flight land before the CTA's shared memory is given back
      const long long c0 = clock64();
      while (clock64() - c0 < 2000000LL) __nanosleep(256);
    }
    return;
  }

  // ---- consumers
  pdl_wait(4);
  bool ok = true;
  int g0 = 0;  // tiles of the chunks before this one
#ifdef ROOST_TRACE
  unsigned long long trc[6] = {0, 0, 0, 0, 0, 0};
#endif
  bool seen = false;  // this thread has read the CTA's first descriptor (with clusters its only one: desc[0] stays as it is)
  for (int k = 0; ok; ++k) {
    if (!(ok = mbar_wait_limited(desc_full(k & 1), (uint32_t)(k >> 1) & 1u, abortp, 5, &g_attention_error))) break;
    const DecodeChunk c = desc[k & 1];
    seen = true;
    if (c.b < 0) break;
#ifdef ROOST_TRACE
    if (k == 0) trc[0] = trace_now();   // descriptor and Q here
#endif
    const int rows_total = c.n * group;  // at most 16
    const int pos0 = c.kv_len - c.n;
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      ldmatrix_x4(q_smem + (k & 1) * kQBytes + Tile<D>::offset(lane & 15, kk * 2 + (lane >> 4)), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(desc_empty(k & 1));  // this warp holds the descriptor and the Q fragments in registers
    int qpos[2], qlo[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int pr = (lane >> 2) + r * 8;
      if (pr < rows_total) {
        qpos[r] = pos0 + pr / group;
        qlo[r] = window > 0 ? max(0, qpos[r] - window + 1) : 0;
      } else {
        qpos[r] = -1;
        qlo[r] = 0;
      }
    }
    RowState<D> st;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) st.o[i][0] = st.o[i][1] = st.o[i][2] = st.o[i][3] = 0.f;
    st.m[0] = st.m[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.f;

    for (int i = (warp - g0 % NW + NW) % NW; i < c.ntiles; i += NW) {
      const int g = g0 + i;
      const int stage = g % STAGES;
      // A wait names its phase by parity only, so it must not be asked of a barrier two phases behind. The stage's
      // previous tile (g - STAGES) may belong to another warp, which may not have taken it yet: once it has handed the
      // stage back, the full barrier is in this tile's phase and no earlier one.
      if (g >= STAGES && !(ok = mbar_wait_limited(empty_bar(stage), (uint32_t)((g / STAGES) - 1) & 1u, abortp, 3, &g_attention_error))) break;
      if (!(ok = mbar_wait_limited(full_bar(stage), (uint32_t)(g / STAGES) & 1u, abortp, 2, &g_attention_error))) break;
      const uint32_t k_tile = smem_base + stage * kStageBytes, v_tile = k_tile + L::kValues;
      const int j0 = (c.t0 + i) * TK;
      if (j0 < c.lo || j0 + TK - 1 > c.hi) {
        // value rows outside the visible keys: zero, so that whatever the pool holds there cannot reach the product
        for (int idx = lane; idx < TK * (D / 8); idx += 32) {
          const int r = idx / (D / 8), ch = idx % (D / 8);
          if (j0 + r < c.lo || j0 + r > c.hi) {
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(v_tile + L::offset(r, ch)), "r"(0u) : "memory");
          }
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // ordered before the copy that reuses the stage
        __syncwarp();
      }
      attend_core<D, TK, L>(
          st, [&](int kk, uint32_t& a0, uint32_t& a1, uint32_t& a2, uint32_t& a3) { a0 = qf[kk][0]; a1 = qf[kk][1]; a2 = qf[kk][2]; a3 = qf[kk][3]; },
          k_tile, v_tile, j0, qpos, qlo, scale_log2, lane);
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(stage));
    }
    g0 += c.ntiles;
#ifdef ROOST_TRACE
    if (k == 0) trc[1] = trace_now();   // this warp's tiles are done
#endif

    // merge the warps' states through shared memory (in warp order), MR packed rows a pass, and write the chunk's result
    for (int r0 = 0; r0 < rows_total; r0 += MR) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int row = (lane >> 2) + r * 8;
        if (row >= r0 && row < r0 + MR && row < rows_total) {
          float* dst = sm_o + ((size_t)warp * MR + (row - r0)) * kScratchStride + (lane & 3) * 2;
#pragma unroll
          for (int nn = 0; nn < D / 8; ++nn) {
            dst[nn * 8] = st.o[nn][2 * r];
            dst[nn * 8 + 1] = st.o[nn][2 * r + 1];
          }
          if ((lane & 3) == 0) {
            sm_ml[(warp * MR + (row - r0)) * 2] = st.m[r];
            sm_ml[(warp * MR + (row - r0)) * 2 + 1] = st.l[r];
          }
        }
      }
      asm volatile("bar.sync 1, %0;\n" ::"n"(NW * 32) : "memory");
      const int pass_rows = min(MR, rows_total - r0);
      for (int idx = tid; idx < pass_rows * D; idx += NW * 32) {
        const int pr = idx / D, col = idx % D;
        const int row = r0 + pr;
        float m = -INFINITY;
#pragma unroll
        for (int ww = 0; ww < NW; ++ww) m = fmaxf(m, sm_ml[(ww * MR + pr) * 2]);
        const float msafe = m == -INFINITY ? 0.f : m;
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int ww = 0; ww < NW; ++ww) {
          const float fac = exp2f(sm_ml[(ww * MR + pr) * 2] - msafe);
          l += sm_ml[(ww * MR + pr) * 2 + 1] * fac;
          o += sm_o[((size_t)ww * MR + pr) * kScratchStride + col] * fac;
        }
        if (cluster_chunks > 0) {
          // a cluster's results: [16][D] sums and [16][2] (maximum, sum of weights) in the first stage of the ring, which
          // no copy writes any more once the CTA's only chunk has been consumed
          float* cl_o = reinterpret_cast<float*>(smem_gen);
          cl_o[row * D + col] = o;
          if (col == 0) {
            cl_o[16 * D + row * 2] = m;
            cl_o[16 * D + row * 2 + 1] = l;
          }
        } else if (c.slot < 0) {
          const float inv = l > 0.f ? 1.0f / l : 0.f;
          out[((size_t)(c.q_start + row / group) * q_heads + c.kvh * group + row % group) * D + col] = __float2bfloat16_rn(o * inv);
        } else {
          const size_t prow = ((size_t)c.slot * kv_heads + c.kvh) * 16 + row;
          part_o[prow * D + col] = o;
          if (col == 0) {
            part_ml[prow * 2] = m;
            part_ml[prow * 2 + 1] = l;
          }
        }
      }
      asm volatile("bar.sync 1, %0;\n" ::"n"(NW * 32) : "memory");  // the scratch (and the Q tile) may be written again
    }
  }
#ifdef ROOST_TRACE
  trc[2] = trace_now();   // the CTA's result is in shared memory (or memory)
#endif
  const bool cl_padding = seen && desc[0].b < 0;  // the cluster's items are padding: all its CTAs leave at once
  if (cluster_chunks > 0 && !cl_padding) {
    const int cl_rows = seen ? desc[0].n * group : 0, cl_q_start = desc[0].q_start, cl_kvh = desc[0].kvh;
    // Every CTA of the cluster has an item of the same row (padding fills whole clusters), so all of them come here, a
    // CTA whose wait was given up included: its numbers are wrong (or, if it never saw its item, it merges nothing), the
    // fault is recorded, and nobody is left waiting or reads the shared memory of a CTA that has gone.
    decode_cluster_sync();  // the results of all the cluster's CTAs are in their shared memory
#ifdef ROOST_TRACE
    trc[3] = trace_now();
#endif
    {  // every CTA of the cluster combines its share of the row's values
      constexpr int kMaxCluster = 8;
      const uint32_t o_addr = smem_base, ml_addr = smem_base + 16 * D * 4;
      for (int idx = tid + (int)decode_cluster_rank() * NW * 32; idx < cl_rows * D; idx += NW * 32 * cluster_chunks) {
        const int row = idx / D, col = idx % D;
        // every load first (they are independent trips to the other CTAs' shared memory), then the sums in chunk order,
        // as the merge kernel forms them
        float pm[kMaxCluster], pl[kMaxCluster], po[kMaxCluster];
#pragma unroll
        for (int cc = 0; cc < kMaxCluster; ++cc) {
          const bool in = cc < cluster_chunks;
          pm[cc] = in ? ld_cluster_f32(ml_addr + (row * 2) * 4, cc) : -INFINITY;
          pl[cc] = in ? ld_cluster_f32(ml_addr + (row * 2 + 1) * 4, cc) : 0.f;
          po[cc] = in ? ld_cluster_f32(o_addr + (row * D + col) * 4, cc) : 0.f;
        }
        float m = -INFINITY;
#pragma unroll
        for (int cc = 0; cc < kMaxCluster; ++cc) m = fmaxf(m, pm[cc]);
        const float msafe = m == -INFINITY ? 0.f : m;
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int cc = 0; cc < kMaxCluster; ++cc) {
          if (cc < cluster_chunks) {
            const float f = exp2f(pm[cc] - msafe);
            l += pl[cc] * f;
            o += po[cc] * f;
          }
        }
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        out[((size_t)(cl_q_start + row / group) * q_heads + cl_kvh * group + row % group) * D + col] = __float2bfloat16_rn(o * inv);
      }
    }
#ifdef ROOST_TRACE
    trc[4] = trace_now();
#endif
    decode_cluster_sync();  // nobody leaves while another CTA still reads its shared memory
#ifdef ROOST_TRACE
    trc[5] = trace_now();
    if (tid == 0 && (blockIdx.x & 7) == 0) trace_flush(4 * 4 + 3, blockIdx.x * 16 + 4, trc, 6);
#endif
  }
  if (!ok) {  // a copy that was waited for in vain may still land
    const long long c0 = clock64();
    while (clock64() - c0 < 2000000LL) __nanosleep(256);
  }
}

constexpr int kMergeAhead = 9;  // chunks whose partial results a merge thread loads in one go (a context of 4096 to 4608 keys)

// merge_work[i] = (batch row, first partial slot, number of chunks | packed rows << 24, the row's first token)
template <int D>
__global__ void attention_merge_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       const int4* __restrict__ merge_work, int q_heads, int kv_heads, int slot_limit) {
  pdl_launch_dependents(5);
  const int4 w = merge_work[blockIdx.x];  // the step's work lists are on the device before the step's first kernel runs
  const int b = w.x, slot0 = w.y, chunks = w.z & 0xffffff, rows_total = w.z >> 24, q_start = w.w;
  pdl_wait(5);
  if (b < 0) return;  // padding of a fixed-size work list
  if (slot0 < 0 || chunks > slot_limit - slot0) {  // the row's partial slots do not all lie in the workspace: see the decode kernel
    if (threadIdx.x == 0) atomicCAS(&g_attention_error, 0, 9);
    return;
  }
  const int kvh = blockIdx.y;
  const int group = q_heads / kv_heads;
  const size_t stride = (size_t)kv_heads * 16;  // partial rows from one chunk's slot to the next
  for (int row = blockIdx.z; row < rows_total; row += gridDim.z) {
    const size_t pr0 = ((size_t)slot0 * kv_heads + kvh) * 16 + row;
    const size_t out_at = ((size_t)(q_start + row / group) * q_heads + kvh * group + row % group) * D;
    if (chunks <= kMergeAhead) {
      // the usual case: every partial maximum, sum and output value this thread needs is loaded at once (one trip to
      // memory instead of two), then combined in chunk order
      float pm[kMergeAhead], pl[kMergeAhead], po[(D + 127) / 128][kMergeAhead];
#pragma unroll
      for (int c = 0; c < kMergeAhead; ++c) {
        if (c < chunks) {
          const size_t pr = pr0 + c * stride;
          const float2 ml = *reinterpret_cast<const float2*>(part_ml + pr * 2);
          pm[c] = ml.x;
          pl[c] = ml.y;
#pragma unroll
          for (int j = 0; j < (D + 127) / 128; ++j) {
            const int col = threadIdx.x + j * 128;
            po[j][c] = col < D ? part_o[pr * D + col] : 0.f;
          }
        } else {
          pm[c] = -INFINITY;
          pl[c] = 0.f;
#pragma unroll
          for (int j = 0; j < (D + 127) / 128; ++j) po[j][c] = 0.f;
        }
      }
      float m = -INFINITY;
#pragma unroll
      for (int c = 0; c < kMergeAhead; ++c) m = fmaxf(m, pm[c]);
      const float msafe = m == -INFINITY ? 0.f : m;
      float l = 0.f, o[(D + 127) / 128];
#pragma unroll
      for (int j = 0; j < (D + 127) / 128; ++j) o[j] = 0.f;
#pragma unroll
      for (int c = 0; c < kMergeAhead; ++c) {  // chunk order: the sums do not depend on how the chunks were scheduled
        if (c < chunks) {
          const float f = exp2f(pm[c] - msafe);
          l += pl[c] * f;
#pragma unroll
          for (int j = 0; j < (D + 127) / 128; ++j) o[j] += po[j][c] * f;
        }
      }
      const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
      for (int j = 0; j < (D + 127) / 128; ++j) {
        const int col = threadIdx.x + j * 128;
        if (col < D) out[out_at + col] = __float2bfloat16_rn(o[j] * inv);
      }
      continue;
    }
    float m = -INFINITY;
#pragma unroll 8
    for (int c = 0; c < chunks; ++c) m = fmaxf(m, part_ml[(pr0 + c * stride) * 2]);
    const float msafe = m == -INFINITY ? 0.f : m;
    for (int col = threadIdx.x; col < D; col += blockDim.x) {
      float l = 0.f, o = 0.f;
#pragma unroll 8
      for (int c = 0; c < chunks; ++c) {  // chunk order: the sums do not depend on how the chunks were scheduled
        const size_t pr = pr0 + c * stride;
        const float f = exp2f(part_ml[pr * 2] - msafe);
        l += part_ml[pr * 2 + 1] * f;
        o += part_o[pr * D + col] * f;
      }
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      out[out_at + col] = __float2bfloat16_rn(o * inv);
    }
  }
}

// attention_tc.cu
bool prefill_tc_serves(int head_dim, int q_heads, int kv_heads, int page_size, long long pool_pages, const void* k_pool, const void* v_pool,
                       const void* q);
int launch_prefill_tc(const void* q, long long tokens, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr,
                      const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work, int items, int tile_rows,
                      int q_heads, int kv_heads, int head_dim, int page_size, long long pool_pages, float scale, int window, cudaStream_t s);
void set_prefill_tc(bool on);
int prefill_tc_status();

static int page_shift_of(int page_size) {
  if (page_size & (page_size - 1)) return -1;
  int s = 0;
  while ((1 << s) < page_size) ++s;
  return s;
}

// A prefill warp carries one or two row tiles of 16. Two halve the shared-memory traffic per product, which pays once the
// grid fills the device several times over; with less work the smaller tiles spread it over more SMs. Both compute a row
// with the same operations in the same order, so the choice does not show in the result.
constexpr int kPrefillWideMinRows = 65536;  // packed rows x key/value heads from which 128-row tiles are used
// ... from which a work item of the tcgen05 kernel is two row groups (256 packed rows): one group's products then run
// while the other's softmax does, which pays once there are enough items for every SM (measured at 32/8 heads of 128, one
// group against two: 1024 tokens 22 against 28 us, 1536 tokens 40 against 37 us, 2048 tokens 58 against 49 us, 4096
// tokens 181 against 146 us)
constexpr int kPrefillTwoGroupsMinRows = 49152;

template <int D, int MT>
static int launch_prefill(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr, const int32_t* kv_lens,
                          const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work, int items, int q_heads, int kv_heads,
                          int page_size, float scale, int window, cudaStream_t s) {
  const size_t smem = (size_t)(64 * MT + 4 * 64) * D * 2;
  auto kernel = attention_prefill_kernel<D, MT>;
  static bool attr_set = false;  // once per process: nothing but launches happens on later calls (stream capture)
  if (smem > 48 * 1024 && !attr_set) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attr_set = true;
  }
  launch_kernel(kernel, dim3(items, kv_heads), dim3(128), smem, s, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_pool,
                (const __nv_bfloat16*)v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, (const int2*)work, q_heads, kv_heads, page_size,
                page_shift_of(page_size), scale * kLog2e, window);
  return check_launch("attention_prefill");
}

static bool g_decode_tma = true;

// Whether the copy-engine decode kernel serves these sizes: head sizes whose rows are whole 128-byte swizzle spans, pages
// of 16, 32, 64, ... rows (a power of two), keys and values in one allocation (the values after the keys, so that one
// tensor map covers both), a pool whose rows fit a tensor map.
static bool decode_tma_serves(int head_dim, int page_size, long long pool_pages, int kv_heads, const void* k_pool, const void* v_pool) {
  if (!g_decode_tma || pool_pages <= 0 || (head_dim != 64 && head_dim != 128)) return false;
  if (page_size < 16 || (page_size & (page_size - 1)) != 0) return false;
  if (pool_pages * kv_heads * page_size >= (1LL << 31)) return false;
  const long long pool_bytes = pool_pages * kv_heads * page_size * head_dim * 2;
  const long long gap = (const char*)v_pool - (const char*)k_pool;
  if (gap < pool_bytes || gap % 16 != 0 || gap >= (1LL << 40)) return false;
  return (uintptr_t)k_pool % 128 == 0 && encode_tiled() != nullptr;
}

// Both pools [pages, kv_heads, page_size, D] as one tensor: 64 columns x pool rows x D / 64 column blocks x {keys, values},
// in boxes of one page's (or 32) rows of both.
static int make_pool_map(CUtensorMap* map, const void* k_pool, const void* v_pool, long long rows, int head_dim, int box_rows) {
  const cuuint64_t dims[4] = {64u, (cuuint64_t)rows, (cuuint64_t)head_dim / 64, 2u};
  const cuuint64_t strides[3] = {(cuuint64_t)head_dim * 2, 128u, (cuuint64_t)((const char*)v_pool - (const char*)k_pool)};
  const cuuint32_t box[4] = {64u, (cuuint32_t)box_rows, (cuuint32_t)head_dim / 64, 2u};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  const CUresult r = encode_tiled()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(k_pool), dims, strides, box, elem,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ROOST_ERR_CUDA, "attention_decode: cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return ROOST_OK;
}

template <int D>
static int launch_decode_tma(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr, const int32_t* kv_lens,
                             const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work, int items, float* part_o,
                             float* part_ml, int q_heads, int kv_heads, int page_size, long long pool_pages, float scale, int window,
                             cudaStream_t s, int cluster_chunks) {
  CUtensorMap map;
  const int box_rows = page_size < kTmaTileKeys ? page_size : kTmaTileKeys;
  const int rc = make_pool_map(&map, k_pool, v_pool, pool_pages * kv_heads * page_size, D, box_rows);
  if (rc != ROOST_OK) return rc;
  constexpr size_t smem = (size_t)tma_decode_stages<D>() * 2 * kTmaTileKeys * D * 2 + 2 * 16 * D * 2 +
                          (size_t)kTmaConsumers * kTmaMergeRows * (D + 8 + 2) * 4 + 1024;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(attention_decode_tma_kernel<D, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(attention_decode_tma_kernel<D, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  const long long total = (long long)items * kv_heads;
  // two CTAs fit an SM; with clusters every CTA takes exactly one item
  const int grid = (int)(cluster_chunks > 0 || total < 2LL * sms ? total : 2LL * sms);
  auto kernel = box_rows == 16 ? attention_decode_tma_kernel<D, 16> : attention_decode_tma_kernel<D, 32>;
  launch_kernel_cluster(kernel, dim3(grid), dim3((kTmaConsumers + 1) * 32), smem, s, cluster_chunks > 0 ? cluster_chunks : 1, map,
                        (const __nv_bfloat16*)q, (__nv_bfloat16*)out, q_indptr, kv_lens, kv_indptr, kv_indices, (const int4*)work, items, part_o,
                        part_ml, q_heads, kv_heads, page_size, scale * kLog2e, window, cluster_chunks);
  return check_launch("attention_decode_tma");
}

template <int D>
static int launch_decode(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr, const int32_t* kv_lens,
                         const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work, int items, const int32_t* merge_work,
                         int merge_items, int merge_rows, float* part_o, float* part_ml, int q_heads, int kv_heads, int page_size,
                         long long pool_pages, float scale, int window, cudaStream_t s, int slot_limit = kNoSlotLimit) {
  int rc = ROOST_OK;
  bool launched = false;
  if constexpr (D == 64 || D == 128) {
    if (slot_limit == kNoSlotLimit && decode_tma_serves(D, page_size, pool_pages, kv_heads, k_pool, v_pool)) {
      rc = launch_decode_tma<D>(q, out, k_pool, v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, work, items, part_o, part_ml, q_heads,
                                kv_heads, page_size, pool_pages, scale, window, s, 0);
      launched = true;
    }
  }
  if (!launched) {
    constexpr int NW = 4;
    const size_t smem = (size_t)16 * D * 2 + (size_t)NW * kDecodeStages * 2 * kDecodeTileKeys * D * 2;
    auto kernel = attention_decode_kernel<D, NW>;
    static bool attr_set[64] = {};   // per device: the attribute belongs to the kernel as loaded on that device
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || !attr_set[dev])) {
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    launch_kernel(kernel, dim3(items, kv_heads), dim3(NW * 32), smem, s, (const __nv_bfloat16*)q, (__nv_bfloat16*)out,
                  (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, (const int4*)work, part_o,
                  part_ml, q_heads, kv_heads, page_size, page_shift_of(page_size), scale * kLog2e, window, slot_limit);
    rc = check_launch("attention_decode");
  }
  if (rc != ROOST_OK || merge_items == 0) return rc;
  const int rows = merge_rows < 1 ? 1 : (merge_rows > 16 ? 16 : merge_rows);  // blocks along z; each walks the rows beyond
  launch_kernel(attention_merge_kernel<D>, dim3(merge_items, kv_heads, rows), dim3(D < 128 ? D : 128), 0, s, (__nv_bfloat16*)out,
                (const float*)part_o, (const float*)part_ml, (const int4*)merge_work, q_heads, kv_heads, slot_limit);
  return check_launch("attention_merge");
}

}  // namespace roost

using namespace roost;

#define ROOST_DISPATCH_HEAD_DIM(d, D, ...)                \
  switch (d) {                                            \
    case 16: { constexpr int D = 16; __VA_ARGS__; } break;   \
    case 32: { constexpr int D = 32; __VA_ARGS__; } break;   \
    case 64: { constexpr int D = 64; __VA_ARGS__; } break;   \
    case 128: { constexpr int D = 128; __VA_ARGS__; } break; \
    case 256: { constexpr int D = 256; __VA_ARGS__; } break; \
    default: return fail(ROOST_ERR_UNSUPPORTED, "attention_mma: head_dim is not one of 16, 32, 64, 128, 256"); \
  }

// Packed rows of one prefill work item for these sizes and pools and a step that brings `packed_rows` packed rows
// (tokens x query heads per key/value head) in all to the prefill kernels: 128 where the tcgen05 kernel serves (or the
// grid of the mma.sync kernel is large), else 64; 0 for a head size no tensor-core kernel serves.
extern "C" int roost_attention_prefill_tile_rows(int head_dim, int q_heads, int kv_heads, int page_size, long long pool_pages,
                                                 const void* k_pool, const void* v_pool, long long packed_rows) {
  if (!roost_attention_mma_supported(head_dim)) return 0;
  if (prefill_tc_serves(head_dim, q_heads, kv_heads, page_size, pool_pages, k_pool, v_pool, nullptr)) {
    // two row groups a CTA keep the tensor cores busy while the other group's softmax runs; with little work the
    // smaller items spread over more SMs
    return packed_rows * kv_heads >= kPrefillTwoGroupsMinRows ? 256 : 128;
  }
  return head_dim <= 128 && packed_rows * kv_heads >= kPrefillWideMinRows ? 128 : 64;
}

// 1: prompt portions run the tcgen05 kernel where the sizes allow (the default); 0: always the mma.sync kernel.
extern "C" void roost_attention_set_prefill_tc(int on) { set_prefill_tc(on != 0); }

// 1: decode rows stream keys and values through the copy engine where the sizes allow (the default); 0: always cp.async.
extern "C" void roost_attention_set_decode_tma(int on) { g_decode_tma = on != 0; }

// 0, or the code of the first wait a decode kernel gave up since the last call (1, 3: a free stage; 2: a tile's copies;
// 4, 5: the chunk descriptors).
namespace roost {
int* attention_error_address() {
  int* p = nullptr;
  return cudaGetSymbolAddress((void**)&p, g_attention_error) == cudaSuccess ? p : nullptr;
}
}  // namespace roost

extern "C" int roost_attention_status(void) {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_attention_error, sizeof(int)) != cudaSuccess) return -1;
  if (code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_attention_error, &zero, sizeof(int));
  }
  const int tc = prefill_tc_status();  // codes of the tcgen05 prefill kernel come back as 100 + code
  if (code == 0 && tc != 0) code = tc < 0 ? tc : 100 + tc;
  return code;
}

extern "C" int roost_attention_mma_supported(int head_dim) {
  return head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256;
}

extern "C" int roost_attention_prefill(const void* q, long long tokens, void* out, const void* k_pool, const void* v_pool,
                                       const int32_t* q_indptr, const int32_t* kv_lens, const int32_t* kv_indptr,
                                       const int32_t* kv_indices, const int32_t* work, int items, int tile_rows, int q_heads, int kv_heads,
                                       int head_dim, int page_size, long long pool_pages, float scale, int window, roost_stream_t stream) {
  ROOST_REQUIRE(items >= 0 && q_heads > 0 && kv_heads > 0 && page_size > 0, "attention_prefill: sizes must be positive");
  ROOST_REQUIRE(tile_rows == 64 || ((tile_rows == 128 || tile_rows == 256) && head_dim <= 128),
                "attention_prefill: a work item has 64 packed rows, or 128 or 256 up to head size 128");
  ROOST_REQUIRE(q_heads % kv_heads == 0, "attention_prefill: q_heads must be a multiple of kv_heads");
  if (kv_heads > 65535) return fail(ROOST_ERR_UNSUPPORTED, "attention_prefill: more than 65535 key/value heads");
  if (items == 0) return ROOST_OK;
  if ((tile_rows == 128 || tile_rows == 256) && tokens > 0 &&
      prefill_tc_serves(head_dim, q_heads, kv_heads, page_size, pool_pages, k_pool, v_pool, q)) {
    return launch_prefill_tc(q, tokens, out, k_pool, v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, work, items, tile_rows, q_heads, kv_heads,
                             head_dim, page_size, pool_pages, scale, window, (cudaStream_t)stream);
  }
  if (tile_rows == 128) {
    switch (head_dim) {
      case 16: return launch_prefill<16, 2>(q, out, k_pool, v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, work, items, q_heads, kv_heads, page_size, scale, window, (cudaStream_t)stream);
      case 32: return launch_prefill<32, 2>(q, out, k_pool, v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, work, items, q_heads, kv_heads, page_size, scale, window, (cudaStream_t)stream);
      case 64: return launch_prefill<64, 2>(q, out, k_pool, v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, work, items, q_heads, kv_heads, page_size, scale, window, (cudaStream_t)stream);
      case 128: return launch_prefill<128, 2>(q, out, k_pool, v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, work, items, q_heads, kv_heads, page_size, scale, window, (cudaStream_t)stream);
      default: return fail(ROOST_ERR_UNSUPPORTED, "attention_prefill: no tensor-core kernel for this head size");
    }
  }
  ROOST_DISPATCH_HEAD_DIM(head_dim, D, return launch_prefill<D, 1>(q, out, k_pool, v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, work, items,
                                                                    q_heads, kv_heads, page_size, scale, window, (cudaStream_t)stream));
  return ROOST_OK;
}

extern "C" int roost_attention_decode(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr,
                                      const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work,
                                      int items, const int32_t* merge_work, int merge_items, int merge_rows, float* part_o, float* part_ml,
                                      int q_heads, int kv_heads, int head_dim, int page_size, long long pool_pages, float scale, int window,
                                      roost_stream_t stream) {
  ROOST_REQUIRE(items >= 0 && merge_items >= 0 && q_heads > 0 && kv_heads > 0 && page_size > 0, "attention_decode: sizes must be positive");
  ROOST_REQUIRE(q_heads % kv_heads == 0, "attention_decode: q_heads must be a multiple of kv_heads");
  ROOST_REQUIRE(merge_items == 0 || (part_o && part_ml && merge_work), "attention_decode: the workspace for split rows is missing");
  if (kv_heads > 65535) return fail(ROOST_ERR_UNSUPPORTED, "attention_decode: more than 65535 key/value heads");
  if (items == 0) return ROOST_OK;
  ROOST_DISPATCH_HEAD_DIM(head_dim, D, return launch_decode<D>(q, out, k_pool, v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, work, items,
                                                                merge_work, merge_items, merge_rows, part_o, part_ml, q_heads, kv_heads,
                                                                page_size, pool_pages, scale, window, (cudaStream_t)stream));
  return ROOST_OK;
}

// ------------------------------------------------------------------------------------------------ no-allocation variant
// roost_attention_decode_static: the split decode attention for callers that cannot give it a workspace.
// (This entry point has no counterpart in the reference; see its declaration in roost_kernels.h.)
//
// Some hosts of this library may not allocate device memory while they run: a server that handed the whole GPU to
// its own arena at start-up and has nothing left for cudaMalloc, a step loop that must never synchronise the device
// (cudaMalloc and cudaFree do), a plug-in that is forbidden to grow its process's footprint. For them the partial
// results of the split rows live in the fixed array below instead of caller-provided buffers. Every process that
// loads the library holds the array on every GPU it touches, until it exits.
namespace roost {

extern "C" int roost_attention_decode_cluster_supported(int head_dim, int page_size, long long pool_pages, int kv_heads, const void* k_pool,
                                                        const void* v_pool) {
  return decode_tma_serves(head_dim, page_size, pool_pages, kv_heads, k_pool, v_pool) ? 1 : 0;
}

extern "C" int roost_attention_decode_cluster(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr,
                                              const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices,
                                              const int32_t* work, int items, int cluster_chunks, int q_heads, int kv_heads, int head_dim,
                                              int page_size, long long pool_pages, float scale, int window, roost_stream_t stream) {
  ROOST_REQUIRE(items >= 0 && q_heads > 0 && kv_heads > 0 && page_size > 0, "attention_decode_cluster: sizes must be positive");
  ROOST_REQUIRE(q_heads % kv_heads == 0, "attention_decode_cluster: q_heads must be a multiple of kv_heads");
  ROOST_REQUIRE(cluster_chunks == 1 || cluster_chunks == 2 || cluster_chunks == 4 || cluster_chunks == 8,
                "attention_decode_cluster: a cluster has 1, 2, 4 or 8 CTAs");
  ROOST_REQUIRE(items % cluster_chunks == 0, "attention_decode_cluster: the work list holds cluster_chunks items a row");
  if ((long long)items * kv_heads >= (1LL << 31)) return fail(ROOST_ERR_UNSUPPORTED, "attention_decode_cluster: too many work items");
  if (!decode_tma_serves(head_dim, page_size, pool_pages, kv_heads, k_pool, v_pool)) {
    return fail(ROOST_ERR_UNSUPPORTED, "attention_decode_cluster: these sizes or pools are not served (see roost_attention_decode_cluster_supported)");
  }
  if (items == 0) return ROOST_OK;
  const cudaStream_t s = (cudaStream_t)stream;
  if (head_dim == 64) {
    return launch_decode_tma<64>(q, out, k_pool, v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, work, items, nullptr, nullptr, q_heads,
                                 kv_heads, page_size, pool_pages, scale, window, s, cluster_chunks);
  }
  return launch_decode_tma<128>(q, out, k_pool, v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, work, items, nullptr, nullptr, q_heads,
                                kv_heads, page_size, pool_pages, scale, window, s, cluster_chunks);
}

constexpr size_t kStaticScratchFloats = 4u * 1024u * 1024u;  // 16 MiB
static __device__ __align__(256) float g_decode_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
static float* g_decode_scratch_ptr[kMaxDevices];  // device addresses of the array, per device; null until set up

// In host code g_decode_scratch is only a handle for the runtime, not an address a kernel may use: the device address
// comes from cudaGetSymbolAddress, asked once per device with that device current.
static int static_scratch(float** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(ROOST_ERR_CUDA, std::string("attention_decode_static: cudaGetDevice: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(ROOST_ERR_UNSUPPORTED, "attention_decode_static: device ordinal beyond 63");
  if (g_decode_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_decode_scratch);
    if (e != cudaSuccess || p == nullptr) {
      return fail(ROOST_ERR_CUDA, std::string("attention_decode_static: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
    }
    g_decode_scratch_ptr[dev] = p;
  }
  *ptr = g_decode_scratch_ptr[dev];
  return ROOST_OK;
}

}  // namespace roost

extern "C" int roost_attention_decode_static_capacity_floats(void) { return (int)kStaticScratchFloats; }

extern "C" int roost_attention_decode_static(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr,
                                             const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices,
                                             const int32_t* work, int items, const int32_t* merge_work, int merge_items, int slots,
                                             int q_heads, int kv_heads, int head_dim, int page_size, float scale, int window,
                                             roost_stream_t stream) {
  ROOST_REQUIRE(items >= 0 && merge_items >= 0 && slots >= 0 && q_heads > 0 && kv_heads > 0 && page_size > 0 && head_dim > 0,
                "attention_decode_static: sizes must be positive");
  ROOST_REQUIRE(q_heads % kv_heads == 0, "attention_decode_static: q_heads must be a multiple of kv_heads");
  ROOST_REQUIRE(merge_items == 0 || merge_work != nullptr, "attention_decode_static: merge_work is null");
  if (kv_heads > 65535) return fail(ROOST_ERR_UNSUPPORTED, "attention_decode_static: more than 65535 key/value heads");
  // partial outputs first, then (max, sum) pairs, the second region starting on a 256-byte boundary
  const size_t o_floats = (size_t)slots * kv_heads * 16 * head_dim;
  const size_t o_padded = (o_floats + 63) / 64 * 64;
  const size_t ml_floats = (size_t)slots * kv_heads * 16 * 2;
  if (o_padded + ml_floats > kStaticScratchFloats) {
    return fail(ROOST_ERR_UNSUPPORTED, "attention_decode_static: " + std::to_string(slots) + " partial slots need " +
                                           std::to_string((o_padded + ml_floats) * 4) + " bytes of scratch; the fixed array holds " +
                                           std::to_string(kStaticScratchFloats * 4) + " (use roost_attention_decode with a workspace)");
  }
  if (items == 0) return ROOST_OK;
  float* scratch = nullptr;
  const int rc = static_scratch(&scratch);
  if (rc != ROOST_OK) return rc;
  // `slots` is also the limit the kernels hold the work lists to: an item that names a slot at or beyond it is skipped
  // (its output rows stay unwritten) and roost_attention_status() reports code 9, so a work list that disagrees with
  // `slots` cannot make the kernels write past the library's array into whatever lies behind it.
  // Nothing in the array has to start at zero: the decode kernel writes every element of a slot that the merge kernel
  // reads (all rows below the request's packed-row count, for every key/value head), so what an earlier call left
  // behind is never read.
  ROOST_DISPATCH_HEAD_DIM(head_dim, D, return launch_decode<D>(q, out, k_pool, v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, work, items,
                                                                merge_work, merge_items, 16, scratch, scratch + o_padded, q_heads, kv_heads,
                                                                page_size, /*pool_pages unknown: the cp.async kernel*/ 0, scale, window,
                                                                (cudaStream_t)stream, /*slot_limit*/ slots));
  return ROOST_OK;
}

ROOST_TRACE_TU(attention_mma)
