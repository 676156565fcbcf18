// out[m,n] = sum_k a[m,k] * w[n,k] in bfloat16 with 32-bit accumulation on the fifth-generation tensor cores:
// TMA loads into 128-byte-swizzled shared memory, tcgen05.mma with the accumulator in tensor memory, a persistent
// warp-specialised kernel. Definition of the result: src/Starlings.Roost.Ops/CpuOps.cs:395-437 (TransposeB, alpha 1, no
// bias, 32-bit accumulation, one rounding); the reference calls cuBLASLt here (kernels/src/gemm.cu:235) and has no
// Blackwell kernel of its own.
//
// One CTA per SM walks output tiles of 128 x 256 (m fastest, so neighbouring CTAs share a tile of w). Roles:
//   warp 0, one lane: producer. Per k-block of 64 it waits for a free stage, arms the stage's barrier with the byte
//     count and issues two TMA loads (a: 128 x 64, w: 256 x 64). Rows beyond m, n or k are zero-filled by the TMA unit.
//   warp 1, one lane: issues four tcgen05.mma (128 x 256 x 16) per k-block into one of two accumulators of 256 tensor
//     memory columns; tcgen05.commit hands the stage back to the producer and, after the last k-block, the accumulator
//     to the epilogue.
//   warps 2..5: epilogue. Each reads its 32 lanes of the accumulator (tcgen05.ld), rounds to the output type and stores
//     rows of 32 columns; the other accumulator is being filled meanwhile.
// Every wait on a barrier is bounded: a wait that does not complete within about a tenth of a second raises an abort
// flag that every role polls, the kernel records an error code, lets copies in flight land, frees its tensor memory and
// returns. roost_gemm_tcgen05_status() reads the code back.
#include <map>
#include <tuple>

#include "tcgen05.cuh"

namespace roost {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int kUmmaK = 16;
constexpr uint32_t kStageABytes = BM * BK * 2;
constexpr uint32_t kStageBBytes = BN * BK * 2;
constexpr uint32_t kStageBytes = kStageABytes + kStageBBytes;
constexpr uint32_t kTmemCols = 512;  // two accumulators of BN columns

__device__ int g_gemm_tcgen05_error = 0;

// ------------------------------------------------------------------------------------------------ PTX wrappers
template <bool CLUSTER = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
  return mbar_wait_limited<CLUSTER>(bar, parity, abort_flag, code, &g_gemm_tcgen05_error);
}
// The pair form: the barrier may live in the other CTA of the pair (a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int c_inner, int c_outer) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(c_inner), "r"(c_outer)
      : "memory");
}
template <typename TOut>
__device__ __forceinline__ void store_row32(TOut* dst, const uint32_t (&v)[32], int valid_cols, bool vec_ok);

template <>
__device__ __forceinline__ void store_row32<__nv_bfloat16>(__nv_bfloat16* dst, const uint32_t (&v)[32], int valid_cols, bool vec_ok) {
  if (valid_cols >= 32 && vec_ok) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t p[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(v[i * 8 + 2 * j]), __uint_as_float(v[i * 8 + 2 * j + 1]));
        p[j] = *reinterpret_cast<uint32_t*>(&b);
      }
      *reinterpret_cast<uint4*>(dst + i * 8) = make_uint4(p[0], p[1], p[2], p[3]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid_cols) dst[i] = __float2bfloat16_rn(__uint_as_float(v[i]));
  }
}
template <>
__device__ __forceinline__ void store_row32<float>(float* dst, const uint32_t (&v)[32], int valid_cols, bool vec_ok) {
  if (valid_cols >= 32 && vec_ok) {
#pragma unroll
    for (int i = 0; i < 8; ++i) *reinterpret_cast<uint4*>(dst + i * 4) = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid_cols) dst[i] = __uint_as_float(v[i]);
  }
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + expf(-g)); }

// EPI 0: out = acc. EPI 1 (SwiGLU): w's rows come in blocks of 256, 128 gate rows followed by the 128 up rows of the same
// outputs, so a tile's columns 0..127 are gate and 128..255 the matching up values: out[m, n0/2 + j] = silu(gate_j) * up_j,
// and out has n/2 columns.
template <typename TOut, int EPI>
__global__ void __launch_bounds__(192, 1)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, TOut* __restrict__ out, int M,
                        int N, int K, int64_t ldo) {
  extern __shared__ unsigned char smem_raw[];
  // tiles want 1024-byte alignment (the swizzle pattern repeats every 1024 bytes)
  const uint32_t smem_base = ((uint32_t)__cvta_generic_to_shared(smem_raw) + 1023u) & ~1023u;
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto acc_empty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 4);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"((uint32_t)__cvta_generic_to_shared(&tmem_base_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abortp = &abort_flag;

  const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  const int k_blocks = (K + BK - 1) / BK;
  const int tiles = m_tiles * n_tiles;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
        const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abortp, 1))) break;
          const uint32_t sa = smem_base + stage * kStageBytes;
          mbar_expect_tx(full_bar(stage), kStageBytes);
          tma_load_2d(sa, &tma_a, full_bar(stage), kb * BK, m0);
          tma_load_2d(sa + kStageABytes, &tma_b, full_bar(stage), kb * BK, n0);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
        if (!(ok = mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, abortp, 2))) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(full_bar(stage), phase, abortp, 3))) break;
          tcgen05_fence_after();
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint64_t a_desc = umma_desc_k_major_sw128(sa);
          const uint64_t b_desc = umma_desc_k_major_sw128(sa + kStageABytes);
#pragma unroll
          for (int k = 0; k < BK / kUmmaK; ++k) {
            // inside the 128-byte swizzle row a step of 16 elements is 32 bytes: two 16-byte units of the address field
            tcgen05_mma_f16(tmem_d, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tcgen05_commit(empty_bar(stage));  // the stage is free once these products have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tcgen05_commit(acc_full_bar(acc));
      }
    }
  } else {
    // epilogue warps 2..5; warp w may read tensor-memory lanes 32 * (w % 4) .. + 31
    const int lane_group = warp & 3;
    const bool vec_ok = (ldo * (int64_t)sizeof(TOut)) % 16 == 0 && ((uintptr_t)out % 16) == 0;
    bool ok = true;
    int it = 0;
    for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
      const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
      if (!(ok = mbar_wait(acc_full_bar(acc), acc_phase, abortp, 4))) break;
      tcgen05_fence_after();
      const int row = m0 + lane_group * 32 + lane;
      if (EPI == 0) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tcgen05_ld_32x32b_x32(tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * BN + c * 32), v);
          const int col = n0 + c * 32;
          if (row < M && col < N) store_row32<TOut>(out + (size_t)row * ldo + col, v, N - col, vec_ok);
        }
      } else {
        const int n_out = N / 2;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t g[32], u[32];
          tcgen05_ld_32x32b_x32(tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * BN + c * 32), g);
          tcgen05_ld_32x32b_x32(tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * BN + BN / 2 + c * 32), u);
#pragma unroll
          for (int i = 0; i < 32; ++i) g[i] = __float_as_uint(silu_f(__uint_as_float(g[i])) * __uint_as_float(u[i]));
          const int col = n0 / 2 + c * 32;
          if (row < M && col < n_out) store_row32<TOut>(out + (size_t)row * ldo + col, g, n_out - col, vec_ok);
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(acc));
    }
  }

  // common exit: on an abort give copies in flight time to land before shared memory is released
  __syncwarp();
  if (*abortp) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(256);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ CTA pairs
// The same product with two CTAs (a cluster of two SMs) on one 256 x 256 tile: tcgen05.mma.cta_group::2 multiplies the
// pair's 256 rows of a by 256 rows of w, of which each CTA stages its own 128 rows of a and 128 rows of w, so a CTA
// fills half as much shared memory per product as in the single-CTA kernel and six stages fit. The even CTA of the pair
// issues every product. Both CTAs' TMA loads count their bytes on the even CTA's barrier (the cta_group::2 form of the
// load allows a barrier in the peer), and the even CTA's tcgen05.commit releases the stage in both CTAs (a multicast
// arrive). Each CTA's epilogue reads its own 128 lanes of tensor memory and tells the even CTA when the
// accumulator is free again. No TMA load is multicast. Waits are bounded as above; the pair meets on the cluster barrier
// before tensor memory is freed.
constexpr int STAGES2 = 6;
constexpr uint32_t kStage2ABytes = 128 * BK * 2;
constexpr uint32_t kStage2BBytes = 128 * BK * 2;
constexpr uint32_t kStage2Bytes = kStage2ABytes + kStage2BBytes;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;  // the barrier at this offset in both CTAs of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::"r"(bar), "h"(mask)
               : "memory");
}
__device__ __forceinline__ void tcgen05_mma_f16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d), "l"(a_desc),
      "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <typename TOut, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
    gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, TOut* __restrict__ out,
                             int M, int N, int K, int64_t ldo) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = ((uint32_t)__cvta_generic_to_shared(smem_raw) + 1023u) & ~1023u;
  // full, empty, peer_full per stage; acc_full, acc_empty per accumulator
  __shared__ __align__(8) uint64_t bars[3 * STAGES2 + 4];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES2 + s); };
  auto peer_full_bar = [&](int s) { return bar0 + 8u * (2 * STAGES2 + s); };
  auto acc_full_bar = [&](int a) { return bar0 + 8u * (3 * STAGES2 + a); };
  auto acc_empty_bar = [&](int a) { return bar0 + 8u * (3 * STAGES2 + 2 + a); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(peer_full_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 8);  // four epilogue warps in each CTA of the pair
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"((uint32_t)__cvta_generic_to_shared(&tmem_base_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anyone arrives on the other's
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abortp = &abort_flag;

  const int m_tiles = (M + 255) / 256, n_tiles = (N + BN - 1) / BN;
  const int k_blocks = (K + BK - 1) / BK;
  const int tiles = m_tiles * n_tiles;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t leader_full[STAGES2];
#pragma unroll
      for (int s2 = 0; s2 < STAGES2; ++s2) leader_full[s2] = mapa_shared(full_bar(s2), 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < tiles && ok; t += pairs) {
        const int m0 = (t % m_tiles) * 256 + (int)rank * 128, n0 = (t / m_tiles) * BN + (int)rank * 128;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abortp, 1))) break;
          const uint32_t sa = smem_base + stage * kStage2Bytes;
          // both CTAs' loads count on the even CTA's barrier, which expects the bytes of both
          if (leader) mbar_expect_tx(full_bar(stage), 2 * kStage2Bytes);
          const uint32_t bar = leader_full[stage];
          tma_load_2d_pair(sa, &tma_a, bar, kb * BK, m0);
          tma_load_2d_pair(sa + kStage2ABytes, &tma_b, bar, kb * BK, n0);
          if (++stage == STAGES2) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = umma_idesc_bf16(256, BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int t = pair; t < tiles && ok; t += pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
        if (!(ok = mbar_wait<true>(acc_empty_bar(acc), acc_phase ^ 1u, abortp, 2))) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait<true>(full_bar(stage), phase, abortp, 3))) break;
          tcgen05_fence_after();
          const uint32_t sa = smem_base + stage * kStage2Bytes;
          const uint64_t a_desc = umma_desc_k_major_sw128(sa);
          const uint64_t b_desc = umma_desc_k_major_sw128(sa + kStage2ABytes);
#pragma unroll
          for (int k = 0; k < BK / kUmmaK; ++k) {
            tcgen05_mma_f16_pair(tmem_d, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tcgen05_commit_pair(empty_bar(stage));  // frees the stage in both CTAs once these products have read it
          if (++stage == STAGES2) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tcgen05_commit_pair(acc_full_bar(acc));
      }
    }
  } else {
    const int lane_group = warp & 3;
    const bool vec_ok = (ldo * (int64_t)sizeof(TOut)) % 16 == 0 && ((uintptr_t)out % 16) == 0;
    const uint32_t leader_acc_empty[2] = {mapa_shared(acc_empty_bar(0), 0), mapa_shared(acc_empty_bar(1), 0)};
    bool ok = true;
    int it = 0;
    for (int t = pair; t < tiles && ok; t += pairs, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
      const int m0 = (t % m_tiles) * 256 + (int)rank * 128, n0 = (t / m_tiles) * BN;
      if (!(ok = mbar_wait(acc_full_bar(acc), acc_phase, abortp, 4))) break;
      tcgen05_fence_after();
      const int row = m0 + lane_group * 32 + lane;
      if (EPI == 0) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tcgen05_ld_32x32b_x32(tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * BN + c * 32), v);
          const int col = n0 + c * 32;
          if (row < M && col < N) store_row32<TOut>(out + (size_t)row * ldo + col, v, N - col, vec_ok);
        }
      } else {
        const int n_out = N / 2;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t g[32], u[32];
          tcgen05_ld_32x32b_x32(tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * BN + c * 32), g);
          tcgen05_ld_32x32b_x32(tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * BN + BN / 2 + c * 32), u);
#pragma unroll
          for (int i = 0; i < 32; ++i) g[i] = __float_as_uint(silu_f(__uint_as_float(g[i])) * __uint_as_float(u[i]));
          const int col = n0 / 2 + c * 32;
          if (row < M && col < n_out) store_row32<TOut>(out + (size_t)row * ldo + col, g, n_out - col, vec_ok);
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_acc_empty[acc]);
    }
  }

  __syncwarp();
  if (*abortp) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(256);
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees shared or tensor memory the other may still be using
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ few rows: weight streaming
// out[m,n] = sum_k x[m,k] * w[n,k] for at most 64 rows of x (decode steps). The work is reading w once at memory speed,
// so the operands swap roles: 128 rows of w are the 128-row operand of tcgen05.mma, the rows of x (padded to 16, 32 or 64)
// its columns, and the accumulator holds out transposed, [128 rows of w] x [rows of x]. One persistent CTA per SM; the
// units of work are (128 rows of w) x (64 of k), 16 KB of w each, and CTA c takes the contiguous range of units
// [c U / G, (c + 1) U / G): every SM streams the same number of bytes, whatever n and k are. A CTA's range covers parts
// of one to three 128-row tiles. A part that is a whole tile is written straight to out. Otherwise the CTA that holds the
// tile's first k-blocks (it reaches them at the END of its range) finishes the tile: the CTAs holding the later k-blocks
// (which they compute at the START of theirs) leave their partial sums in a workspace slot and raise a flag; the finisher
// waits for the flags (a bounded wait), adds the partial sums up in CTA order, adds its own, writes out and lowers the
// flags. The order of every sum is fixed by the geometry alone, so results are the same on every run and for every batch.
// SWIGLU: w's rows come in blocks of 256, 128 gate rows followed by the 128 up rows of the same outputs (the layout of the
// fused product for many rows above). A tile is then such a block, with two accumulators that share the x operand; a row
// of tensor memory holds the gate and the up value of one output, and the CTA that finishes the tile writes
// silu(gate) * up, so out has n / 2 columns.
template <bool SWIGLU>
struct StreamCfg {
  static constexpr int kWRows = SWIGLU ? 256 : 128;           // rows of w in a tile
  static constexpr int kStages = SWIGLU ? 5 : 8;
  static constexpr uint32_t kStageW = kWRows * BK * 2;
  static constexpr uint32_t kStageX = 64 * BK * 2;
  static constexpr uint32_t kStage = kStageW + kStageX;
  static constexpr uint32_t kAccCols = SWIGLU ? 128 : 64;     // tensor-memory columns of one tile's accumulators
  static constexpr int kParts = SWIGLU ? 2 : 1;                // accumulators a tile has
};
constexpr int kStreamMaxCtas = 256;

template <typename TOut, bool SWIGLU>
__global__ void __launch_bounds__(192, 1)
    gemm_stream_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x, TOut* __restrict__ out, int M,
                       int N, int K, int64_t ldo, int ntok, float* ws, int* flags) {
  using Cfg = StreamCfg<SWIGLU>;
  constexpr int STAGES_S = Cfg::kStages;
  constexpr uint32_t kStageSWBytes = Cfg::kStageW, kStageSBytes = Cfg::kStage;
  constexpr int WR = Cfg::kWRows;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = ((uint32_t)__cvta_generic_to_shared(smem_raw) + 1023u) & ~1023u;
  __shared__ __align__(8) uint64_t bars[2 * STAGES_S + 4];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES_S + s); };
  auto acc_full_bar = [&](int a) { return bar0 + 8u * (2 * STAGES_S + a); };
  auto acc_empty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES_S + 2 + a); };
  constexpr uint32_t kCols = 2 * Cfg::kAccCols;  // two tiles' accumulators

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (N + WR - 1) / WR;
  const int kbs = (K + BK - 1) / BK;
  const long long units = (long long)n_tiles * kbs;
  const int G = gridDim.x, c = blockIdx.x;
  const long long u0 = units * c / G, u1 = units * (c + 1) / G;
  const int t_first = (int)(u0 / kbs), t_last = (int)((u1 - 1) / kbs);  // u1 > u0: the host launches at most `units` CTAs
  int prologue = 0;  // units whose loads the producer issued before the CTA-wide barrier
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tma_w)) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tma_x)) : "memory");
    abort_flag = 0;
    for (int s = 0; s < STAGES_S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    // the first stages are free by construction: the loads of w start now (no kernel writes the weights), while tensor
    // memory is still being allocated and, under programmatic dependent launch, while the kernel that produces x is still
    // running; the loads of x follow once that kernel has finished
    pdl_launch_dependents(6);
    for (long long u = u0; u < u1 && prologue < STAGES_S; ++u, ++prologue) {
      const int t = (int)(u / kbs), kb = (int)(u % kbs);
      const uint32_t sw = smem_base + prologue * kStageSBytes;
      mbar_expect_tx(full_bar(prologue), kStageSWBytes + (uint32_t)ntok * BK * 2);
      tma_load_2d(sw, &tma_w, full_bar(prologue), kb * BK, t * WR);
    }
    pdl_wait(6);
    for (int i = 0; i < prologue; ++i) {
      const int kb = (int)((u0 + i) % kbs);
      tma_load_2d(smem_base + i * kStageSBytes + kStageSWBytes, &tma_x, full_bar(i), kb * BK, 0);
    }
  } else {
    pdl_wait();  // every thread that later reads what earlier kernels wrote (workspace, flags) has waited
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"((uint32_t)__cvta_generic_to_shared(&tmem_base_slot)),
                 "r"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      int stage = prologue % STAGES_S;
      uint32_t phase = prologue == STAGES_S ? 1u : 0u;
      bool ok = true;
      for (long long u = u0 + prologue; u < u1 && ok; ++u) {
        const int t = (int)(u / kbs), kb = (int)(u % kbs);
        if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abortp, 1))) break;
        const uint32_t sw = smem_base + stage * kStageSBytes;
        mbar_expect_tx(full_bar(stage), kStageSWBytes + (uint32_t)ntok * BK * 2);
        tma_load_2d(sw, &tma_w, full_bar(stage), kb * BK, t * WR);
        tma_load_2d(sw + kStageSWBytes, &tma_x, full_bar(stage), kb * BK, 0);
        if (++stage == STAGES_S) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(128, ntok);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
#ifdef ROOST_TRACE
      unsigned long long tr_mma[2] = {0, 0};
#endif
      for (int t = t_first; t <= t_last && ok; ++t, ++it) {
        const long long s0 = max(u0, (long long)t * kbs), s1 = min(u1, (long long)(t + 1) * kbs);
        const int acc = it & 1;
        const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
        if (!(ok = mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, abortp, 2))) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)acc * Cfg::kAccCols;
        for (long long u = s0; u < s1; ++u) {
          if (!(ok = mbar_wait(full_bar(stage), phase, abortp, 3))) break;
          tcgen05_fence_after();
#ifdef ROOST_TRACE
          if (u == u0) tr_mma[0] = trace_now();
#endif
          const uint32_t sw = smem_base + stage * kStageSBytes;
          const uint64_t a_desc = umma_desc_k_major_sw128(sw);
          const uint64_t b_desc = umma_desc_k_major_sw128(sw + kStageSWBytes);
#pragma unroll
          for (int k = 0; k < BK / kUmmaK; ++k) {
            tcgen05_mma_f16(tmem_d, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc, (u > s0 || k > 0) ? 1u : 0u);
            if constexpr (SWIGLU) {  // the up rows, 128 rows (16 KB) further down the stage
              tcgen05_mma_f16(tmem_d + 64, a_desc + (uint64_t)(2 * k) + (uint64_t)((128 * BK * 2) >> 4), b_desc + (uint64_t)(2 * k), idesc,
                              (u > s0 || k > 0) ? 1u : 0u);
            }
          }
          tcgen05_commit(empty_bar(stage));
          if (++stage == STAGES_S) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tcgen05_commit(acc_full_bar(acc));
      }
#ifdef ROOST_TRACE
      tr_mma[1] = trace_now();
      trace_flush(6 * 4 + 3, blockIdx.x * 8, tr_mma, 2);
#endif
    }
  } else {
    const int lane_group = warp & 3;
    const int etid = (warp - 2) * 32 + lane;  // 0..127 among the epilogue threads
#ifdef ROOST_TRACE
    unsigned long long tr_epi[3] = {0, 0, 0};
#endif
    bool ok = true;
    int it = 0;
    for (int t = t_first; t <= t_last && ok; ++t, ++it) {
      const long long s0 = max(u0, (long long)t * kbs), s1 = min(u1, (long long)(t + 1) * kbs);
      const int k0 = (int)(s0 - (long long)t * kbs), k1 = (int)(s1 - (long long)t * kbs);
      const int acc = it & 1;
      const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
      constexpr int P = Cfg::kParts;         // accumulators of a tile: the product, or gate and up
      constexpr int QMAX = SWIGLU ? 2 : 4;   // sixteen-column groups of x rows this variant serves
      const int r = lane_group * 32 + lane;  // row within the tile's accumulators = lane of tensor memory
      const int n = t * 128 + r;             // column of out
      const int n_out = SWIGLU ? N / 2 : N;
      const uint32_t taddr = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(acc * Cfg::kAccCols);
      if (k0 > 0) {
        // a later part of the tile: leave the partial sums for the CTA that holds the tile's first k-blocks
        if (!(ok = mbar_wait(acc_full_bar(acc), acc_phase, abortp, 4))) break;
        tcgen05_fence_after();
#pragma unroll
        for (int p = 0; p < P; ++p) {
          for (int cb = 0; cb < ntok; cb += 16) {
            uint32_t v[16];
            tcgen05_ld_32x32b_x16(taddr + p * 64 + cb, v);
#pragma unroll
            for (int i = 0; i < 16; ++i) ws[(((size_t)c * P + p) * 64 + cb + i) * 128 + r] = __uint_as_float(v[i]);
          }
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;\n" ::: "memory");  // the four epilogue warps
        if (etid == 0) {
          __threadfence();
          atomicExch(&flags[c], 1);
        }
      } else {
        // the tile's first part: a whole tile, or the finisher of a tile that continues in the next CTAs. Those CTAs
        // reach their part of this tile first of all, so their partial sums are often there before this CTA's own
        // accumulator is: they are fetched and added up (in CTA order) while the tensor cores still work on it.
        int contributors = 0;
        float psum[P][QMAX][16];
        if (k1 < kbs) {
          long long covered = s1;
          while (covered < (long long)(t + 1) * kbs && c + 1 + contributors < G) {
            ++contributors;
            covered = units * (c + 1 + contributors) / G;
          }
          if (etid < contributors) {
            const long long w0 = clock64();
            while (atomicAdd(&flags[c + 1 + etid], 0) == 0) {
              if (*abortp || clock64() - w0 > kWaitCycles) {
                *abortp = 1;
                atomicCAS(&g_gemm_tcgen05_error, 0, 7);
                break;
              }
            }
            __threadfence();
          }
          asm volatile("bar.sync 1, 128;\n" ::: "memory");
#pragma unroll
          for (int p = 0; p < P; ++p) {
#pragma unroll
            for (int q = 0; q < QMAX; ++q) {
              if (q * 16 < ntok) {
#pragma unroll
                for (int i = 0; i < 16; ++i) psum[p][q][i] = 0.f;
                for (int j0 = 0; j0 < contributors; j0 += 4) {  // the loads of four contributors are in flight together
                  float part[4][16];
#pragma unroll
                  for (int jj = 0; jj < 4; ++jj) {
                    if (j0 + jj < contributors) {
#pragma unroll
                      for (int i = 0; i < 16; ++i) part[jj][i] = __ldcg(&ws[(((size_t)(c + 1 + j0 + jj) * P + p) * 64 + q * 16 + i) * 128 + r]);
                    }
                  }
#pragma unroll
                  for (int jj = 0; jj < 4; ++jj) {
                    if (j0 + jj < contributors) {
#pragma unroll
                      for (int i = 0; i < 16; ++i) psum[p][q][i] += part[jj][i];
                    }
                  }
                }
              }
            }
          }
        }
#ifdef ROOST_TRACE
        tr_epi[0] = trace_now();
#endif
        if (!(ok = mbar_wait(acc_full_bar(acc), acc_phase, abortp, 4))) break;
        tcgen05_fence_after();
#ifdef ROOST_TRACE
        tr_epi[1] = trace_now();
#endif
#pragma unroll
        for (int q = 0; q < QMAX; ++q) {
          if (q * 16 < ntok) {
            uint32_t v[P][16];
#pragma unroll
            for (int p = 0; p < P; ++p) tcgen05_ld_32x32b_x16(taddr + p * 64 + q * 16, v[p]);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int m = q * 16 + i;
              float val[P];
#pragma unroll
              for (int p = 0; p < P; ++p) val[p] = contributors > 0 ? __uint_as_float(v[p][i]) + psum[p][q][i] : __uint_as_float(v[p][i]);
              const float res = SWIGLU ? silu_f(val[0]) * val[P - 1] : val[0];
              if (m < M && n < n_out) out[(size_t)m * ldo + n] = from_float<TOut>(res);
            }
          }
        }
        if (contributors > 0) {
          asm volatile("bar.sync 1, 128;\n" ::: "memory");
          if (etid < contributors) atomicExch(&flags[c + 1 + etid], 0);  // lowered for the next launch
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(acc));
    }
#ifdef ROOST_TRACE
    tr_epi[2] = trace_now();
    if (etid == 0) trace_flush(6 * 4 + 3, blockIdx.x * 8 + 2, tr_epi, 3);
#endif
  }

  trace_point(6, 2);
  __syncwarp();
  if (*abortp) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(256);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kCols) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ few rows: k split over a cluster
// The same product for shapes with few 128-row tiles of w and a long k (the attention's output projection, the down
// projection): the grid is thread-block clusters of `split` CTAs, one cluster a tile, CTA r of a cluster taking the r-th
// part of k. Two CTAs fit an SM and every CTA asks for all its first stages of w at once, before the kernel in front has
// finished, so nearly the whole matrix is on its way when the product starts. The partial sums never go to memory:
// every CTA leaves its accumulator in its own shared memory, and after a cluster barrier CTA r adds up, in CTA order, the
// r-th part of the tile's rows through distributed shared memory and writes it. The order of every sum is fixed by
// (n, k) alone, so results are the same on every run and for every batch.
constexpr int kSplitMaxStages = 6;

__device__ __forceinline__ float ld_dsmem_f32(uint32_t addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote));
  return v;
}
// Every thread of the cluster that has not exited arrives and waits; the threads of a warp need not come together.
__device__ __forceinline__ void cluster_sync_unaligned() {
  asm volatile("barrier.cluster.arrive.release;\nbarrier.cluster.wait.acquire;\n" ::: "memory");
}

// SWIGLU: w's rows come in blocks of 256 (128 gate rows, then the 128 up rows of the same outputs), a tile is such a
// block with two accumulators that share the x operand, and what is written is silu(gate) * up: out has n / 2 columns.
template <typename TOut, bool SWIGLU>
__global__ void __launch_bounds__(192, 2)
    gemm_split_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x, TOut* __restrict__ out, int M,
                      int N, int K, int64_t ldo, int ntok, int split, int stages) {
  constexpr int WR = SWIGLU ? 256 : 128;  // rows of w in a tile
  constexpr int P = SWIGLU ? 2 : 1;       // accumulators of a tile
  const uint32_t stage_w = WR * BK * 2, stage_bytes = stage_w + (uint32_t)ntok * BK * 2;  // a multiple of 1024 bytes
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = ((uint32_t)__cvta_generic_to_shared(smem_raw) + 1023u) & ~1023u;
  float* red = reinterpret_cast<float*>(smem_raw + (smem_base - (uint32_t)__cvta_generic_to_shared(smem_raw)));  // [P][m][128], over the first stages
  __shared__ __align__(8) uint64_t bars[2 * kSplitMaxStages + 1];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kSplitMaxStages + s); };
  const uint32_t acc_full_bar = bar0 + 8u * (2 * kSplitMaxStages);
  const uint32_t acc_cols = ntok <= 32 ? 32u : 64u;   // tensor-memory columns of one accumulator
  const uint32_t tmem_cols = acc_cols * P;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x / split, r = blockIdx.x % split;  // the cluster's tile; this CTA's rank in the cluster
  const int kbs = (K + BK - 1) / BK;
  const int kb0 = (int)((long long)kbs * r / split), kb1 = (int)((long long)kbs * (r + 1) / split);  // kb1 > kb0: kbs >= split
  int prologue = 0;
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tma_w)) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tma_x)) : "memory");
    abort_flag = 0;
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    pdl_launch_dependents(7);
    // no kernel writes the weights: their loads start while the kernel that produces x is still running
    for (int kb = kb0; kb < kb1 && prologue < stages; ++kb, ++prologue) {
      mbar_expect_tx(full_bar(prologue), stage_bytes);
      tma_load_2d(smem_base + prologue * stage_bytes, &tma_w, full_bar(prologue), kb * BK, t * WR);
    }
    pdl_wait(7);
    for (int i = 0; i < prologue; ++i) tma_load_2d(smem_base + i * stage_bytes + stage_w, &tma_x, full_bar(i), (kb0 + i) * BK, 0);
  } else {
    pdl_wait();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"((uint32_t)__cvta_generic_to_shared(&tmem_base_slot)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abortp = &abort_flag;
#ifdef ROOST_TRACE
  unsigned long long tr[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  tr[0] = trace_now();   // set-up done: barriers, tensor memory, the CTA-wide barrier
#endif

  if (warp == 0) {
    if (lane == 0) {
      int stage = prologue % stages;
      uint32_t phase = prologue == stages ? 1u : 0u;
      bool ok = true;
      for (int kb = kb0 + prologue; kb < kb1 && ok; ++kb) {
        if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abortp, 1))) break;
        const uint32_t sw = smem_base + stage * stage_bytes;
        mbar_expect_tx(full_bar(stage), stage_bytes);
        tma_load_2d(sw, &tma_w, full_bar(stage), kb * BK, t * WR);
        tma_load_2d(sw + stage_w, &tma_x, full_bar(stage), kb * BK, 0);
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(128, ntok);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1 && ok; ++kb) {
        if (!(ok = mbar_wait(full_bar(stage), phase, abortp, 3))) break;
        tcgen05_fence_after();
#ifdef ROOST_TRACE
        if (kb == kb0) tr[1] = trace_now();   // the first stage has landed
#endif
        const uint32_t sw = smem_base + stage * stage_bytes;
        const uint64_t a_desc = umma_desc_k_major_sw128(sw);
        const uint64_t b_desc = umma_desc_k_major_sw128(sw + stage_w);
#pragma unroll
        for (int k = 0; k < BK / kUmmaK; ++k) {
          tcgen05_mma_f16(tmem_base, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          if constexpr (SWIGLU) {  // the up rows, 128 rows (16 KB) further down the stage
            tcgen05_mma_f16(tmem_base + acc_cols, a_desc + (uint64_t)(2 * k) + (uint64_t)((128 * BK * 2) >> 4), b_desc + (uint64_t)(2 * k), idesc,
                            (kb > kb0 || k > 0) ? 1u : 0u);
          }
        }
        tcgen05_commit(empty_bar(stage));
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) tcgen05_commit(acc_full_bar);
#ifdef ROOST_TRACE
      tr[2] = trace_now();                    // the last products are issued
      if ((blockIdx.x & 7) == 0) trace_flush(7 * 4 + 3, blockIdx.x * 16, tr, 3);
#endif
    }
  } else {
    // the accumulator (out transposed: a lane of tensor memory is a row of the tile, a column a row of x) into this CTA's
    // shared memory as [row of x][128], over the first stages, which no copy writes any more
    const int lane_group = warp & 3;
    const int row = lane_group * 32 + lane;
    if (mbar_wait(acc_full_bar, 0u, abortp, 4)) {
      tcgen05_fence_after();
#ifdef ROOST_TRACE
      tr[3] = trace_now();                    // the accumulator is complete
#endif
      const uint32_t taddr = tmem_base + ((uint32_t)(lane_group * 32) << 16);
#pragma unroll
      for (int p = 0; p < P; ++p) {
        for (int cb = 0; cb < ntok && cb < M; cb += 16) {
          uint32_t v[16];
          tcgen05_ld_32x32b_x16(taddr + p * acc_cols + cb, v);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if (cb + i < M) red[((p * M) + cb + i) * 128 + row] = __uint_as_float(v[i]);
          }
        }
      }
    }
    tcgen05_fence_before();
  }
  // Every thread of every CTA of the cluster comes here, whatever its waits returned: nobody is left waiting at the
  // cluster's barriers and nobody reads the shared memory of a CTA that has gone.
  __syncwarp();
#ifdef ROOST_TRACE
  tr[4] = trace_now();                        // the partial sums are in shared memory
#endif
  cluster_sync_unaligned();  // the partial sums of all the cluster's CTAs are in their shared memory
#ifdef ROOST_TRACE
  tr[5] = trace_now();
#endif
  if (warp >= 2) {
    const int etid = (warp - 2) * 32 + lane;
    const int lo = 128 * r / split, cnt = 128 * (r + 1) / split - lo;  // this CTA's share of the tile's rows
    const uint32_t red_addr = smem_base;
    const int n_out = SWIGLU ? N / 2 : N;
    for (int idx = etid; idx < cnt * M; idx += 128) {
      const int m = idx / cnt, nl = lo + idx % cnt, n = t * 128 + nl;
      float part[P][8];
#pragma unroll
      for (int p = 0; p < P; ++p) {
#pragma unroll
        for (int rr = 0; rr < 8; ++rr) {
          part[p][rr] = rr < split ? ld_dsmem_f32(red_addr + (uint32_t)((p * M + m) * 128 + nl) * 4u, (uint32_t)rr) : 0.f;
        }
      }
      float sum[P];
#pragma unroll
      for (int p = 0; p < P; ++p) {
        sum[p] = part[p][0];
#pragma unroll
        for (int rr = 1; rr < 8; ++rr) {
          if (rr < split) sum[p] += part[p][rr];
        }
      }
      const float res = SWIGLU ? silu_f(sum[0]) * sum[P - 1] : sum[0];
      if (n < n_out) out[(size_t)m * ldo + n] = from_float<TOut>(res);
    }
  }
#ifdef ROOST_TRACE
  tr[6] = trace_now();                        // this CTA's share is written
#endif
  cluster_sync_unaligned();  // nobody leaves while another CTA still reads its shared memory
#ifdef ROOST_TRACE
  tr[7] = trace_now();
  if (threadIdx.x == 64 && (blockIdx.x & 7) == 0) trace_flush(7 * 4 + 3, blockIdx.x * 16 + 3, tr + 3, 5);
#endif
  trace_point(7, 2);
  if (*abortp) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(256);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ host side
// A [rows, k] bfloat16 matrix with row stride ld elements as a 2-D tensor map with boxes of box_rows x 64 elements.
static int make_map(CUtensorMap* map, const void* base, int rows, int k, int64_t ld, int box_rows) {
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return fail(ROOST_ERR_CUDA, "gemm_tcgen05: the driver does not export cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ROOST_ERR_CUDA, "gemm_tcgen05: cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return ROOST_OK;
}

template <typename TOut, int EPI>
static int launch_tcgen05(const CUtensorMap& ma, const CUtensorMap& mb, void* out, int m, int n, int k, int64_t ldo, cudaStream_t s) {
  static int sms = 0;
  static bool attr_set = false;
  const size_t smem = (size_t)STAGES * kStageBytes + 1024;
  auto kernel = gemm_tcgen05_kernel<TOut, EPI>;
  if (!attr_set) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attr_set = true;
  }
  const int tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
  const int grid = tiles < sms ? tiles : sms;
  kernel<<<grid, 192, smem, s>>>(ma, mb, (TOut*)out, m, n, k, ldo);
  return check_launch("gemm_tcgen05");
}

template <typename TOut, int EPI>
static int launch_tcgen05_pair(const CUtensorMap& ma, const CUtensorMap& mb, void* out, int m, int n, int k, int64_t ldo, cudaStream_t s) {
  static int sms = 0;
  static bool attr_set = false;
  const size_t smem = (size_t)STAGES2 * kStage2Bytes + 1024;
  auto kernel = gemm_tcgen05_pair_kernel<TOut, EPI>;
  if (!attr_set) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attr_set = true;
  }
  const int tiles = ((m + 255) / 256) * ((n + BN - 1) / BN);
  int pairs = sms / 2;
  if (tiles < pairs) pairs = tiles;
  kernel<<<2 * pairs, 192, smem, s>>>(ma, mb, (TOut*)out, m, n, k, ldo);
  return check_launch("gemm_tcgen05_pair");
}

template <typename TOut, bool SWIGLU>
static int launch_stream(const CUtensorMap& mw, const CUtensorMap& mx, void* out, int m, int n, int k, int64_t ldo, int ntok, float* ws,
                         int* flags, cudaStream_t s) {
  using Cfg = StreamCfg<SWIGLU>;
  static int sms = 0;
  static bool attr_set = false;
  const size_t smem = (size_t)Cfg::kStages * Cfg::kStage + 1024;
  auto kernel = gemm_stream_kernel<TOut, SWIGLU>;
  if (!attr_set) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attr_set = true;
  }
  const long long units = (long long)((n + Cfg::kWRows - 1) / Cfg::kWRows) * ((k + BK - 1) / BK);
  long long grid = sms < kStreamMaxCtas ? sms : kStreamMaxCtas;
  if (units < grid) grid = units;
  launch_kernel(kernel, dim3((int)grid), dim3(192), smem, s, mw, mx, (TOut*)out, m, n, k, ldo, ntok, ws, flags);
  return check_launch("gemm_stream");
}

// CTAs of a cluster for the k-split product of an [n, k] weight: the most (up to 8) that still lets every cluster run at
// once with two CTAs an SM and leaves every CTA at least two 64-wide blocks of k; 0 when the shape has too many tiles.
static int split_for(int n, int k, int tile_rows = 128) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles = (n + tile_rows - 1) / tile_rows, kbs = (k + BK - 1) / BK;
  int split = (2 * sms) / tiles;
  if (split > 8) split = 8;
  if (split > kbs / 2) split = kbs / 2;
  while (split & (split - 1)) split &= split - 1;  // a power of two: clusters of 2, 4 and 8 fill the SMs of a GPC, 6 and 7 leave some idle
  return split >= 2 ? split : 0;
}

template <typename TOut, bool SWIGLU>
static int launch_split(const CUtensorMap& mw, const CUtensorMap& mx, void* out, int m, int n, int k, int64_t ldo, int ntok, int split,
                        cudaStream_t s) {
  constexpr int WR = SWIGLU ? 256 : 128;
  // At most about 100 KB, so that two CTAs fit an SM. With few rows of x four stages (72 KB) were measured best in the
  // step (4.16 against 4.20 ms with six, 4.17 with three or five): a CTA of the next product then fits beside two of this
  // one and has its weights on the way before these are done.
  // A CTA with a long part of k (the 32B sizes: 32 and 100 blocks) keeps six: 13.82 against 13.93 ms a step there.
  const int blocks_a_cta = ((k + BK - 1) / BK) / split;
  const int stages = SWIGLU ? 3 : (ntok == 16 ? (blocks_a_cta >= 32 ? 6 : 4) : (ntok == 32 ? 5 : 4));
  const size_t smem = (size_t)stages * (WR * BK * 2 + ntok * BK * 2) + 1024;
  auto kernel = gemm_split_kernel<TOut, SWIGLU>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  const int tiles = (n + WR - 1) / WR;
  launch_kernel_cluster(kernel, dim3(tiles * split), dim3(192), smem, s, split, mw, mx, (TOut*)out, m, n, k, ldo, ntok, split, stages);
  return check_launch("gemm_split");
}

static bool g_use_pairs = true;

}  // namespace roost

using namespace roost;

// 1: products run on pairs of CTAs (256 x 256 tiles, tcgen05 cta_group::2); 0: one CTA a tile (128 x 256).
extern "C" void roost_gemm_tcgen05_set_pairs(int on) { g_use_pairs = on != 0; }

extern "C" int roost_gemm_tcgen05_supported(int m, int n, int k, int64_t lda, int64_t ldw) {
  return m >= 1 && n >= 1 && k >= 8 && k % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0;
}

// The error code a kernel recorded when it gave a wait up (0: none), cleared by the call. 1: producer waiting for a free
// stage, 2: issuer waiting for a free accumulator, 3: issuer waiting for a stage's data, 4: epilogue waiting for an
// accumulator. Synchronises the device.
namespace roost {
int* gemm_tcgen05_error_address() {
  int* p = nullptr;
  return cudaGetSymbolAddress((void**)&p, g_gemm_tcgen05_error) == cudaSuccess ? p : nullptr;
}
}  // namespace roost

extern "C" int roost_gemm_tcgen05_status(void) {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_gemm_tcgen05_error, sizeof(int)) != cudaSuccess) return -1;
  if (code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_gemm_tcgen05_error, &zero, sizeof(int));
  }
  return code;
}

extern "C" int roost_gemm_tcgen05(const void* a, const void* w, void* out, int m, int n, int k, int64_t lda, int64_t ldw, int64_t ldo,
                                  int out_dtype, roost_stream_t stream) {
  ROOST_REQUIRE(out_dtype == ROOST_BF16 || out_dtype == ROOST_F32, "gemm_tcgen05: the output is bfloat16 (1) or float32 (0)");
  ROOST_REQUIRE(lda >= k && ldw >= k && ldo >= n, "gemm_tcgen05: a leading dimension is smaller than its row");
  if (!roost_gemm_tcgen05_supported(m, n, k, lda, ldw)) {
    return fail(ROOST_ERR_UNSUPPORTED, "gemm_tcgen05: k and the row strides must be multiples of 8 elements (TMA wants 16-byte strides)");
  }
  ROOST_REQUIRE(((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_tcgen05: a and w must start on 16-byte boundaries");
  CUtensorMap ma, mb;
  int rc = make_map(&ma, a, m, k, lda, BM);
  if (rc != ROOST_OK) return rc;
  rc = make_map(&mb, w, n, k, ldw, g_use_pairs ? 128 : BN);
  if (rc != ROOST_OK) return rc;
  if (g_use_pairs) {
    if (out_dtype == ROOST_BF16) return launch_tcgen05_pair<__nv_bfloat16, 0>(ma, mb, out, m, n, k, ldo, (cudaStream_t)stream);
    return launch_tcgen05_pair<float, 0>(ma, mb, out, m, n, k, ldo, (cudaStream_t)stream);
  }
  if (out_dtype == ROOST_BF16) return launch_tcgen05<__nv_bfloat16, 0>(ma, mb, out, m, n, k, ldo, (cudaStream_t)stream);
  return launch_tcgen05<float, 0>(ma, mb, out, m, n, k, ldo, (cudaStream_t)stream);
}

// a [m, k] times the gate/up weight w [n, k] (n = 2 * inter, rows interleaved in blocks of 128 gate rows then their 128 up
// rows), SiLU(gate) * up applied to the accumulator: out [m, n / 2] bfloat16. The [m, n] product never reaches memory.
extern "C" int roost_gemm_tcgen05_swiglu(const void* a, const void* w, void* out, int m, int n, int k, int64_t lda, int64_t ldw,
                                         int64_t ldo, roost_stream_t stream) {
  ROOST_REQUIRE(lda >= k && ldw >= k && ldo >= n / 2, "gemm_tcgen05_swiglu: a leading dimension is smaller than its row");
  if (!roost_gemm_tcgen05_supported(m, n, k, lda, ldw) || n % 256 != 0) {
    return fail(ROOST_ERR_UNSUPPORTED, "gemm_tcgen05_swiglu: n must be a multiple of 256 (gate and up rows interleaved in blocks of 128), k and the strides multiples of 8");
  }
  ROOST_REQUIRE(((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_tcgen05_swiglu: a and w must start on 16-byte boundaries");
  CUtensorMap ma, mb;
  int rc = make_map(&ma, a, m, k, lda, BM);
  if (rc != ROOST_OK) return rc;
  rc = make_map(&mb, w, n, k, ldw, g_use_pairs ? 128 : BN);
  if (rc != ROOST_OK) return rc;
  if (g_use_pairs) return launch_tcgen05_pair<__nv_bfloat16, 1>(ma, mb, out, m, n, k, ldo, (cudaStream_t)stream);
  return launch_tcgen05<__nv_bfloat16, 1>(ma, mb, out, m, n, k, ldo, (cudaStream_t)stream);
}

// Workspace of the weight-streaming product: floats for the partial sums and ints for the flags (zero before the first
// call; every call leaves them zero).
extern "C" int roost_gemm_stream_workspace_floats(void) { return kStreamMaxCtas * 2 * 64 * 128; }  // two accumulators a CTA
extern "C" int roost_gemm_stream_workspace_flags(void) { return kStreamMaxCtas; }

extern "C" int roost_gemm_stream_supported(int m, int n, int k, int64_t ldx, int64_t ldw) {
  return m >= 1 && m <= 64 && n >= 1 && k >= 8 && k % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0;
}

extern "C" int roost_gemm_stream(const void* x, const void* w, void* out, int m, int n, int k, int64_t ldx, int64_t ldw, int64_t ldo,
                                 int out_dtype, float* ws, int32_t* flags, roost_stream_t stream) {
  ROOST_REQUIRE(out_dtype == ROOST_BF16 || out_dtype == ROOST_F32, "gemm_stream: the output is bfloat16 (1) or float32 (0)");
  ROOST_REQUIRE(ldx >= k && ldw >= k && ldo >= n, "gemm_stream: a leading dimension is smaller than its row");
  ROOST_REQUIRE(ws != nullptr && flags != nullptr, "gemm_stream: the workspace is missing");
  if (!roost_gemm_stream_supported(m, n, k, ldx, ldw)) {
    return fail(ROOST_ERR_UNSUPPORTED, "gemm_stream: needs 1 <= m <= 64, k and the row strides multiples of 8");
  }
  ROOST_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_stream: x and w must start on 16-byte boundaries");
  const int ntok = m <= 16 ? 16 : (m <= 32 ? 32 : 64);
  CUtensorMap mw, mx;
  int rc = make_map(&mw, w, n, k, ldw, 128);
  if (rc != ROOST_OK) return rc;
  rc = make_map(&mx, x, m, k, ldx, ntok);
  if (rc != ROOST_OK) return rc;
  if (out_dtype == ROOST_BF16) return launch_stream<__nv_bfloat16, false>(mw, mx, out, m, n, k, ldo, ntok, ws, flags, (cudaStream_t)stream);
  return launch_stream<float, false>(mw, mx, out, m, n, k, ldo, ntok, ws, flags, (cudaStream_t)stream);
}

extern "C" int roost_gemm_split_supported(int m, int n, int k, int64_t ldx, int64_t ldw) {
  return roost_gemm_stream_supported(m, n, k, ldx, ldw) && split_for(n, k) > 0;
}

// Where the k-split product was measured faster than the library's and than the weight-streaming kernel on a B200: clusters
// of eight, at least four 64-wide blocks of k a CTA, at most 8 rows of x (16 with a k of 8192 or more); clusters of four
// with a k of 8192 or more and at most 8 rows (alone no faster than cuBLAS, in the step it is). For 8 rows:
// [4096, 4096] 10.3 us against 12.3 (cuBLAS) and 12.5 (stream); [4096, 12288] 21.3 against 32.1 and 23.5; [1024, 3072]
// 5.9 against 8.6 and 10.7; but [6144, 4096] 13.4 against 11.8 and [5120, 8192] (clusters of four) 19.0 against 18.3.
extern "C" int roost_gemm_split_preferred(int m, int n, int k, int64_t ldx, int64_t ldw) {
  if (!roost_gemm_split_supported(m, n, k, ldx, ldw)) return 0;
  const int split = split_for(n, k);
  if (split == 4 && k >= 8192 && m <= 8) return 1;  // the 32B sizes' output and down projections: 14.01 -> 13.82 ms a step
  if (split != 8 || k < 2048) return 0;
  return (m <= 8 || (m <= 16 && k >= 8192)) ? 1 : 0;
}

// out = x w^T for at most 64 rows of x and a weight of few 128-row tiles and a long k: k split over thread-block clusters,
// partial sums added up through distributed shared memory (no workspace).
extern "C" int roost_gemm_split(const void* x, const void* w, void* out, int m, int n, int k, int64_t ldx, int64_t ldw, int64_t ldo,
                                int out_dtype, roost_stream_t stream) {
  ROOST_REQUIRE(out_dtype == ROOST_BF16 || out_dtype == ROOST_F32, "gemm_split: the output is bfloat16 (1) or float32 (0)");
  ROOST_REQUIRE(ldx >= k && ldw >= k && ldo >= n, "gemm_split: a leading dimension is smaller than its row");
  if (!roost_gemm_split_supported(m, n, k, ldx, ldw)) {
    return fail(ROOST_ERR_UNSUPPORTED, "gemm_split: needs 1 <= m <= 64, k and the row strides multiples of 8, and few enough tiles for clusters");
  }
  ROOST_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_split: x and w must start on 16-byte boundaries");
  const int ntok = m <= 16 ? 16 : (m <= 32 ? 32 : 64);
  CUtensorMap mw, mx;
  int rc = make_map(&mw, w, n, k, ldw, 128);
  if (rc != ROOST_OK) return rc;
  rc = make_map(&mx, x, m, k, ldx, ntok);
  if (rc != ROOST_OK) return rc;
  const int split = split_for(n, k);
  if (out_dtype == ROOST_BF16) return launch_split<__nv_bfloat16, false>(mw, mx, out, m, n, k, ldo, ntok, split, (cudaStream_t)stream);
  return launch_split<float, false>(mw, mx, out, m, n, k, ldo, ntok, split, (cudaStream_t)stream);
}

extern "C" int roost_gemm_split_swiglu_supported(int m, int n, int k, int64_t ldx, int64_t ldw) {
  return roost_gemm_stream_swiglu_supported(m, n, k, ldx, ldw) && split_for(n, k, 256) > 0;
}

// out[m, j] = silu(gate_j) * up_j for w's rows in blocks of 256 (128 gate rows, then the 128 up rows of the same outputs),
// k split over thread-block clusters; out has n / 2 columns.
extern "C" int roost_gemm_split_swiglu(const void* x, const void* w, void* out, int m, int n, int k, int64_t ldx, int64_t ldw, int64_t ldo,
                                       int out_dtype, roost_stream_t stream) {
  ROOST_REQUIRE(out_dtype == ROOST_BF16 || out_dtype == ROOST_F32, "gemm_split_swiglu: the output is bfloat16 (1) or float32 (0)");
  ROOST_REQUIRE(ldx >= k && ldw >= k && ldo >= n / 2, "gemm_split_swiglu: a leading dimension is smaller than its row");
  if (!roost_gemm_split_swiglu_supported(m, n, k, ldx, ldw)) {
    return fail(ROOST_ERR_UNSUPPORTED, "gemm_split_swiglu: needs 1 <= m <= 32, n a multiple of 256, k and the row strides multiples of 8, and few enough tiles for clusters");
  }
  ROOST_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_split_swiglu: x and w must start on 16-byte boundaries");
  const int ntok = m <= 16 ? 16 : 32;
  CUtensorMap mw, mx;
  int rc = make_map(&mw, w, n, k, ldw, 256);
  if (rc != ROOST_OK) return rc;
  rc = make_map(&mx, x, m, k, ldx, ntok);
  if (rc != ROOST_OK) return rc;
  const int split = split_for(n, k, 256);
  if (out_dtype == ROOST_BF16) return launch_split<__nv_bfloat16, true>(mw, mx, out, m, n, k, ldo, ntok, split, (cudaStream_t)stream);
  return launch_split<float, true>(mw, mx, out, m, n, k, ldo, ntok, split, (cudaStream_t)stream);
}

extern "C" int roost_gemm_stream_swiglu_supported(int m, int n, int k, int64_t ldx, int64_t ldw) {
  return m >= 1 && m <= 32 && n >= 256 && n % 256 == 0 && k >= 8 && k % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0;
}

// out[m, j] = silu(gate_j) * up_j for w's rows in blocks of 256 (128 gate rows, then the 128 up rows of the same outputs);
// out has n / 2 columns.
extern "C" int roost_gemm_stream_swiglu(const void* x, const void* w, void* out, int m, int n, int k, int64_t ldx, int64_t ldw, int64_t ldo,
                                        int out_dtype, float* ws, int32_t* flags, roost_stream_t stream) {
  ROOST_REQUIRE(out_dtype == ROOST_BF16 || out_dtype == ROOST_F32, "gemm_stream_swiglu: the output is bfloat16 (1) or float32 (0)");
  ROOST_REQUIRE(ldx >= k && ldw >= k && ldo >= n / 2, "gemm_stream_swiglu: a leading dimension is smaller than its row");
  ROOST_REQUIRE(ws != nullptr && flags != nullptr, "gemm_stream_swiglu: the workspace is missing");
  if (!roost_gemm_stream_swiglu_supported(m, n, k, ldx, ldw)) {
    return fail(ROOST_ERR_UNSUPPORTED, "gemm_stream_swiglu: needs 1 <= m <= 32, n a multiple of 256, k and the row strides multiples of 8");
  }
  ROOST_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_stream_swiglu: x and w must start on 16-byte boundaries");
  const int ntok = m <= 16 ? 16 : 32;
  CUtensorMap mw, mx;
  int rc = make_map(&mw, w, n, k, ldw, 256);
  if (rc != ROOST_OK) return rc;
  rc = make_map(&mx, x, m, k, ldx, ntok);
  if (rc != ROOST_OK) return rc;
  if (out_dtype == ROOST_BF16) return launch_stream<__nv_bfloat16, true>(mw, mx, out, m, n, k, ldo, ntok, ws, flags, (cudaStream_t)stream);
  return launch_stream<float, true>(mw, mx, out, m, n, k, ldo, ntok, ws, flags, (cudaStream_t)stream);
}

ROOST_TRACE_TU(gemm_tcgen05)
