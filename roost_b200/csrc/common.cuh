// Shared helpers of the kernel library: status reporting, dtype load/store, block reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string>

#include "roost_kernels.h"

namespace roost {

void set_error(const std::string& msg);

// Programmatic dependent launch. A kernel launched through launch_kernel() with the switch on may begin while the kernel
// before it on the stream is still running: what it does before pdl_wait() (index arithmetic, barrier set-up, loads of
// weights, which no kernel writes) overlaps that kernel's tail; pdl_wait() returns once the earlier kernel has finished
// and its writes are visible. pdl_launch_dependents() lets the next kernel start its own preamble. Both are no-ops for a
// kernel launched without the attribute. The switch is process-wide (roost_set_pdl).
extern bool g_pdl_enabled;

// `cluster_x` > 1 launches the grid as thread-block clusters of that many CTAs along x (the grid's x is a multiple of it).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_x,
                                         Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_pdl_enabled ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cluster_x > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)cluster_x;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  return launch_kernel_cluster(kernel, grid, block, smem, stream, 1, args...);
}

}  // namespace roost
// Development builds (-DROOST_TRACE) record device timestamps of kernel phases through trace.cuh; the product build
// compiles none of it and sees the two empty stand-ins below.
#ifdef ROOST_TRACE
#include "trace.cuh"
#endif
namespace roost {
#ifndef ROOST_TRACE
__device__ __forceinline__ void trace_point(int, int) {}
#define ROOST_TRACE_TU(name)
#endif

__device__ __forceinline__ void pdl_wait(int tag = 0) {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  trace_point(tag, 1);
}
__device__ __forceinline__ void pdl_launch_dependents(int tag = 0) {
  trace_point(tag, 0);
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}

inline int fail(int code, const std::string& msg) {
  set_error(msg);
  return code;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    return fail(ROOST_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
  }
  return ROOST_OK;
}

#define ROOST_REQUIRE(cond, msg)                           \
  do {                                                     \
    if (!(cond)) return ::roost::fail(ROOST_ERR_INVALID, (msg)); \
  } while (0)

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Weight vectors (norm weights) may be stored in either dtype whatever the activations are.
__device__ __forceinline__ float load_w(const void* w, int i, int wdtype) {
  return wdtype == ROOST_F32 ? reinterpret_cast<const float*>(w)[i]
                             : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; the order of additions depends on the block size only, so a row's
// result does not depend on which other rows are in the launch. scratch: 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float t = (threadIdx.x < nwarps) ? scratch[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) scratch[0] = t;
  }
  __syncthreads();
  return scratch[0];
}

// 16-byte loads and stores of activations: 8 bfloat16 or 4 float as 32-bit values in registers.
template <typename T>
struct Vec;
template <>
struct Vec<float> {
  static constexpr int N = 4;
  __device__ static __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  __device__ static __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 t = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&b);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

}  // namespace roost

// Dispatch on an activation dtype code.
#define ROOST_DISPATCH_DTYPE(code, T, ...)                                                   \
  do {                                                                                       \
    if ((code) == ROOST_F32) {                                                               \
      using T = float;                                                                       \
      __VA_ARGS__;                                                                           \
    } else if ((code) == ROOST_BF16) {                                                       \
      using T = __nv_bfloat16;                                                               \
      __VA_ARGS__;                                                                           \
    } else {                                                                                 \
      return ::roost::fail(ROOST_ERR_INVALID, "dtype code is neither float32 (0) nor bfloat16 (1)"); \
    }                                                                                        \
  } while (0)
