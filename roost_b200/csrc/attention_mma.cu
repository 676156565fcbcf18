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
//   * prefill: a CTA of 4 warps owns 64 packed rows of one request and one key/value head and walks the keys in
//     tiles of 64, double-buffered with cp.async, all warps sharing each tile;
//   * decode (rows with at most 16 packed rows): a CTA owns one fixed-size chunk of a request's keys; its warps take
//     the chunk's 16-key tiles in turn, each with a three-stage buffer of its own, and merge their partial results in
//     shared memory; a request with several chunks writes (max, sum, unnormalised output) per chunk to a workspace
//     that the merge kernel reduces in chunk order. The chunk size is fixed by the caller, so the order of every sum
//     depends on the request's own length only, never on what else is in the batch.
// Keys outside a request's visible range are never read: their shared-memory rows are zero-filled.
#include "common.cuh"

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

// One warp, 16 query rows (A operand from q_smem rows q_row0..+15), BN keys from a K/V tile: S = Q K^T, online
// softmax, O += P V. qpos/qlo: per held row, the last and first visible key position (qlo > qpos masks the row).
template <int D, int BN>
__device__ __forceinline__ void attend_tile(RowState<D>& st, uint32_t q_smem, int q_row0, uint32_t k_smem, uint32_t v_smem, int j0,
                                            const int (&qpos)[2], const int (&qlo)[2], float scale_log2, int lane) {
  constexpr int NT = BN / 8;
  float s[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a0, a1, a2, a3;
    ldmatrix_x4(q_smem + Tile<D>::offset(q_row0 + (lane & 15), kk * 2 + (lane >> 4)), a0, a1, a2, a3);
#pragma unroll
    for (int n2 = 0; n2 < NT / 2; ++n2) {
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(k_smem + Tile<D>::offset(n2 * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
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
      ldmatrix_x4_trans(v_smem + Tile<D>::offset(kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), n2 * 2 + (lane >> 4)), b0, b1, b2, b3);
      mma_bf16(st.o[2 * n2], a0, a1, a2, a3, b0, b1);
      mma_bf16(st.o[2 * n2 + 1], a0, a1, a2, a3, b2, b3);
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
// work[i] = (batch row, first packed row of the tile)
template <int D>
__global__ void __launch_bounds__(128) attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                                                                const __nv_bfloat16* __restrict__ k_pool,
                                                                const __nv_bfloat16* __restrict__ v_pool,
                                                                const int32_t* __restrict__ q_indptr, const int32_t* __restrict__ kv_lens,
                                                                const int32_t* __restrict__ kv_indptr,
                                                                const int32_t* __restrict__ kv_indices, const int2* __restrict__ work,
                                                                int q_heads, int kv_heads, int page_size, int page_shift, float scale_log2, int window) {
  constexpr int BM = 64, BN = 64, NT = 128;
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

  // this thread's two rows
  int qpos[2], qlo[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int pr = row0 + warp * 16 + (lane >> 2) + r * 8;
    if (pr < rows_total) {
      qpos[r] = pos0 + pr / group;
      qlo[r] = window > 0 ? max(0, qpos[r] - window + 1) : 0;
    } else {
      qpos[r] = -1;  // sees nothing
      qlo[r] = 0;
    }
  }
  // the tile's key range
  const int last_row = min(row0 + BM, rows_total) - 1;
  const int hi = pos0 + last_row / group;
  const int lo = window > 0 ? max(0, pos0 + row0 / group - window + 1) : 0;
  const int t0 = lo / BN, t1 = hi / BN;

  load_q_tile<D, BM, NT>(q_smem, q, q_start, q_heads, group, kvh, row0, rows_total, tid);
  load_kv_tile<D, BN, NT>(k_smem[0], v_smem[0], k_pool, v_pool, pages, page_size, page_shift, kv_heads, kvh, t0 * BN, lo, hi, tid);
  cp_async_commit();

  RowState<D> st;
#pragma unroll
  for (int i = 0; i < D / 8; ++i) st.o[i][0] = st.o[i][1] = st.o[i][2] = st.o[i][3] = 0.f;
  st.m[0] = st.m[1] = -INFINITY;
  st.l[0] = st.l[1] = 0.f;

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
    attend_tile<D, BN>(st, q_smem, warp * 16, k_smem[stage], v_smem[stage], t * BN, qpos, qlo, scale_log2, lane);
    __syncthreads();
  }

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int pr = row0 + warp * 16 + (lane >> 2) + r * 8;
    if (pr >= rows_total) continue;
    const float inv = st.l[r] > 0.f ? 1.0f / st.l[r] : 0.f;
    __nv_bfloat16* dst = out + ((size_t)(q_start + pr / group) * q_heads + kvh * group + pr % group) * D + (lane & 3) * 2;
#pragma unroll
    for (int nn = 0; nn < D / 8; ++nn) {
      *reinterpret_cast<uint32_t*>(dst + nn * 8) = pack_bf16(st.o[nn][2 * r] * inv, st.o[nn][2 * r + 1] * inv);
    }
  }
}

// ------------------------------------------------------------------------------------------------ decode
// work[i] = (batch row, first key of the chunk, one past its last key, partial slot or -1 for a row with one chunk)
// Partial results of slot s and key/value head h: part_o[(s * kv_heads + h) * 16 + row][D], part_ml[...][2].
template <int D, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32)
    attention_decode_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ k_pool,
                            const __nv_bfloat16* __restrict__ v_pool, const int32_t* __restrict__ q_indptr,
                            const int32_t* __restrict__ kv_lens, const int32_t* __restrict__ kv_indptr,
                            const int32_t* __restrict__ kv_indices, const int4* __restrict__ work, float* __restrict__ part_o,
                            float* __restrict__ part_ml, int q_heads, int kv_heads, int page_size, int page_shift, float scale_log2, int window) {
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

  pdl_launch_dependents();
  pdl_wait();
  const int4 w = work[blockIdx.x];
  const int b = w.x, kv_begin = w.y, kv_end = w.z, slot = w.w;
  if (b < 0) return;  // padding of a fixed-size work list
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

// merge_work[i] = (batch row, first partial slot, number of chunks)
template <int D>
__global__ void attention_merge_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       const int32_t* __restrict__ q_indptr, const int4* __restrict__ merge_work, int q_heads,
                                       int kv_heads) {
  pdl_launch_dependents();
  pdl_wait();
  const int4 w = merge_work[blockIdx.x];
  const int b = w.x, slot0 = w.y, chunks = w.z;
  if (b < 0) return;  // padding of a fixed-size work list
  const int kvh = blockIdx.y;
  const int row = blockIdx.z;
  const int group = q_heads / kv_heads;
  const int q_start = q_indptr[b];
  const int rows_total = (q_indptr[b + 1] - q_start) * group;
  if (row >= rows_total) return;
  const size_t pr0 = ((size_t)slot0 * kv_heads + kvh) * 16 + row;
  const size_t stride = (size_t)kv_heads * 16;  // partial rows from one chunk's slot to the next
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
    out[((size_t)(q_start + row / group) * q_heads + kvh * group + row % group) * D + col] = __float2bfloat16_rn(o * inv);
  }
}

static int page_shift_of(int page_size) {
  if (page_size & (page_size - 1)) return -1;
  int s = 0;
  while ((1 << s) < page_size) ++s;
  return s;
}

template <int D>
static int launch_prefill(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr, const int32_t* kv_lens,
                          const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work, int items, int q_heads, int kv_heads,
                          int page_size, float scale, int window, cudaStream_t s) {
  const size_t smem = (size_t)(64 + 4 * 64) * D * 2;
  auto kernel = attention_prefill_kernel<D>;
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

template <int D>
static int launch_decode(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr, const int32_t* kv_lens,
                         const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work, int items, const int32_t* merge_work,
                         int merge_items, float* part_o, float* part_ml, int q_heads, int kv_heads, int page_size, float scale, int window,
                         cudaStream_t s) {
  constexpr int NW = 4;
  const size_t smem = (size_t)16 * D * 2 + (size_t)NW * kDecodeStages * 2 * kDecodeTileKeys * D * 2;
  auto kernel = attention_decode_kernel<D, NW>;
  static bool attr_set = false;
  if (smem > 48 * 1024 && !attr_set) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attr_set = true;
  }
  launch_kernel(kernel, dim3(items, kv_heads), dim3(NW * 32), smem, s, (const __nv_bfloat16*)q, (__nv_bfloat16*)out,
                (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, (const int4*)work, part_o,
                part_ml, q_heads, kv_heads, page_size, page_shift_of(page_size), scale * kLog2e, window);
  int rc = check_launch("attention_decode");
  if (rc != ROOST_OK || merge_items == 0) return rc;
  launch_kernel(attention_merge_kernel<D>, dim3(merge_items, kv_heads, 16), dim3(D < 128 ? D : 128), 0, s, (__nv_bfloat16*)out,
                (const float*)part_o, (const float*)part_ml, q_indptr, (const int4*)merge_work, q_heads, kv_heads);
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

extern "C" int roost_attention_mma_supported(int head_dim) {
  return head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256;
}

extern "C" int roost_attention_prefill(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr,
                                       const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices,
                                       const int32_t* work, int items, int q_heads, int kv_heads, int head_dim, int page_size,
                                       float scale, int window, roost_stream_t stream) {
  ROOST_REQUIRE(items >= 0 && q_heads > 0 && kv_heads > 0 && page_size > 0, "attention_prefill: sizes must be positive");
  ROOST_REQUIRE(q_heads % kv_heads == 0, "attention_prefill: q_heads must be a multiple of kv_heads");
  if (kv_heads > 65535) return fail(ROOST_ERR_UNSUPPORTED, "attention_prefill: more than 65535 key/value heads");
  if (items == 0) return ROOST_OK;
  ROOST_DISPATCH_HEAD_DIM(head_dim, D, return launch_prefill<D>(q, out, k_pool, v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, work, items,
                                                                 q_heads, kv_heads, page_size, scale, window, (cudaStream_t)stream));
  return ROOST_OK;
}

extern "C" int roost_attention_decode(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr,
                                      const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work,
                                      int items, const int32_t* merge_work, int merge_items, float* part_o, float* part_ml, int q_heads,
                                      int kv_heads, int head_dim, int page_size, float scale, int window, roost_stream_t stream) {
  ROOST_REQUIRE(items >= 0 && merge_items >= 0 && q_heads > 0 && kv_heads > 0 && page_size > 0, "attention_decode: sizes must be positive");
  ROOST_REQUIRE(q_heads % kv_heads == 0, "attention_decode: q_heads must be a multiple of kv_heads");
  ROOST_REQUIRE(merge_items == 0 || (part_o && part_ml && merge_work), "attention_decode: the workspace for split rows is missing");
  if (kv_heads > 65535) return fail(ROOST_ERR_UNSUPPORTED, "attention_decode: more than 65535 key/value heads");
  if (items == 0) return ROOST_OK;
  ROOST_DISPATCH_HEAD_DIM(head_dim, D, return launch_decode<D>(q, out, k_pool, v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, work, items,
                                                                merge_work, merge_items, part_o, part_ml, q_heads, kv_heads, page_size,
                                                                scale, window, (cudaStream_t)stream));
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
  // Nothing in the array has to start at zero: the decode kernel writes every element of a slot that the merge kernel
  // reads (all rows below the request's packed-row count, for every key/value head), so what an earlier call left
  // behind is never read.
  ROOST_DISPATCH_HEAD_DIM(head_dim, D, return launch_decode<D>(q, out, k_pool, v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, work, items,
                                                                merge_work, merge_items, scratch, scratch + o_padded, q_heads, kv_heads,
                                                                page_size, scale, window, (cudaStream_t)stream));
  return ROOST_OK;
}
