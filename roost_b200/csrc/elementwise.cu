// Embedding gather, RMS norm (with the residual add fused), SiLU-and-multiply, and the library's status plumbing.
//
// Definitions (what each must compute) follow the reference's plain ops: embedding
// src/Starlings.Roost.Ops/CpuOps.cs:441-458 (a bad id gives a zero row on the device, kernels/src/m0_ops.cu:306-312),
// RMS norm CpuOps.cs:87-101, the fused add + norm CpuOps.Fused.cs:26-34, SiLU-and-multiply CpuOps.cs:355-368.
// Sums of squares, the reciprocal square root, the residual sum and silu are computed in 32-bit.
#include "common.cuh"

namespace roost {

static thread_local std::string g_last_error;
void set_error(const std::string& msg) { g_last_error = msg; }
bool g_pdl_enabled = false;

// ---------------------------------------------------------------------------------------------- embedding
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int32_t* __restrict__ ids, T* __restrict__ out,
                                 int hidden, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  const T* src = table + (size_t)(ok ? id : 0) * hidden;
  T* dst = out + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? src[i] : from_float<T>(0.f);
}

// ---------------------------------------------------------------------------------------------- rms norm
// One block per output row. ADD: s = residual + x, rounded to T, is what gets normed (and written back when
// the rows are not gathered).
template <typename T, bool ADD>
__global__ void rms_norm_kernel(const T* __restrict__ x, T* residual, const void* __restrict__ w, T* __restrict__ out,
                                const int32_t* __restrict__ rows, int hidden, float eps, int wdtype) {
  extern __shared__ float row[];  // hidden floats, then 32 floats of reduction scratch
  float* scratch = row + hidden;
  pdl_launch_dependents();
  pdl_wait();
  const int i_out = blockIdx.x;
  const size_t r = rows ? (size_t)rows[i_out] : (size_t)i_out;
  const T* xr = x + r * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = to_float(xr[i]);
    if (ADD) {
      T s = from_float<T>(v + to_float(residual[r * hidden + i]));
      if (!rows) residual[r * hidden + i] = s;
      v = to_float(s);
    }
    row[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)i_out * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<T>(row[i] * inv * load_w(w, i, wdtype));
}

// ---------------------------------------------------------------------------------------------- silu and multiply
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int inter, int block) {
  const size_t t = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  if (i >= inter) return;
  const size_t g_at = block ? (size_t)(i / block) * 2 * block + i % block : (size_t)i;
  const size_t u_at = block ? g_at + block : (size_t)inter + i;
  const float g = to_float(x[t * 2 * inter + g_at]);
  const float u = to_float(x[t * 2 * inter + u_at]);
  out[t * inter + i] = from_float<T>(g / (1.0f + expf(-g)) * u);
}


// ---------------------------------------------------------------------------------------------- vectorised forms
// 16-byte loads and stores (Vec in common.cuh), the row kept in registers between the sum of squares and the scaling.
// Used when the row length is a multiple of the vector and short enough for kMaxVec vectors a thread.
constexpr int kMaxVec = 4;
constexpr int kNormWideRows = 1024;  // from this many rows on a bfloat16 norm gives a thread four vectors

// N consecutive weights starting at element i (a multiple of N; the vector is then 8-byte aligned at least).
template <int N>
__device__ __forceinline__ void load_w_vec(const void* w, int i, int wdtype, float (&o)[N]) {
  static_assert(N == 4 || N == 8, "vectors of four or eight elements");
  if (wdtype == ROOST_F32) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + i);
#pragma unroll
    for (int k = 0; k < N / 4; ++k) {
      const float4 f = p[k];
      o[4 * k] = f.x; o[4 * k + 1] = f.y; o[4 * k + 2] = f.z; o[4 * k + 3] = f.w;
    }
  } else {
    const uint2* p = reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(w) + i);
#pragma unroll
    for (int k = 0; k < N / 4; ++k) {
      const uint2 u = p[k];
      o[4 * k] = __uint_as_float(u.x << 16); o[4 * k + 1] = __uint_as_float(u.x & 0xffff0000u);
      o[4 * k + 2] = __uint_as_float(u.y << 16); o[4 * k + 3] = __uint_as_float(u.y & 0xffff0000u);
    }
  }
}

// EARLY_W (steps of few rows, where the kernel's latency is its cost): the weights are in registers before the wait for
// the kernel in front; otherwise they are read when they are used, which keeps the registers for more rows in flight.
template <typename T, bool ADD, bool EARLY_W>
__global__ void rms_norm_vec_kernel(const T* __restrict__ x, T* residual, const void* __restrict__ w, T* __restrict__ out,
                                    const int32_t* __restrict__ rows, int hidden, float eps, int wdtype) {
  constexpr int N = Vec<T>::N;
  __shared__ float scratch[32];
  pdl_launch_dependents(1);
  // the weights and the list of rows do not come from the kernel in front: they are read while it finishes
  const int i_out = blockIdx.x;
  const size_t r = rows ? (size_t)rows[i_out] : (size_t)i_out;
  const int nvec = hidden / N;
  float wv[EARLY_W ? kMaxVec : 1][N];
  if constexpr (EARLY_W) {
#pragma unroll
    for (int k = 0; k < kMaxVec; ++k) {
      const int vi = threadIdx.x + k * blockDim.x;
      if (vi < nvec) load_w_vec<N>(w, vi * N, wdtype, wv[k]);
    }
  }
  pdl_wait(1);
  float v[kMaxVec][N];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < kMaxVec; ++k) {
    const int vi = threadIdx.x + k * blockDim.x;
    if (vi < nvec) {
      Vec<T>::load(x + r * hidden + (size_t)vi * N, v[k]);
      if (ADD) {
        float res[N];
        Vec<T>::load(residual + r * hidden + (size_t)vi * N, res);
#pragma unroll
        for (int e = 0; e < N; ++e) v[k][e] = to_float(from_float<T>(v[k][e] + res[e]));  // the sum, rounded once
        if (!rows) Vec<T>::store(residual + r * hidden + (size_t)vi * N, v[k]);
      }
#pragma unroll
      for (int e = 0; e < N; ++e) ss += v[k][e] * v[k][e];
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
  for (int k = 0; k < kMaxVec; ++k) {
    const int vi = threadIdx.x + k * blockDim.x;
    if (vi < nvec) {
      float o[N];
      if constexpr (!EARLY_W) load_w_vec<N>(w, vi * N, wdtype, wv[0]);
#pragma unroll
      for (int e = 0; e < N; ++e) o[e] = v[k][e] * inv * wv[EARLY_W ? k : 0][e];
      Vec<T>::store(out + (size_t)i_out * hidden + (size_t)vi * N, o);
    }
  }
}

// block 0: a row of x is [gate (inter) | up (inter)]; block b > 0: blocks of b gate values followed by their b up values.
template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ x, T* __restrict__ out, int inter, int block) {
  constexpr int N = Vec<T>::N;
  const size_t t = blockIdx.x;
  const int vi = blockIdx.y * blockDim.x + threadIdx.x;
  pdl_launch_dependents(2);
  pdl_wait(2);
  if (vi * N >= inter) return;
  float g[N], u[N], o[N];
  const int j = vi * N;
  const size_t g_at = block ? (size_t)(j / block) * 2 * block + j % block : (size_t)j;
  const size_t u_at = block ? g_at + block : (size_t)inter + j;
  Vec<T>::load(x + t * 2 * inter + g_at, g);
  Vec<T>::load(x + t * 2 * inter + u_at, u);
#pragma unroll
  for (int e = 0; e < N; ++e) o[e] = g[e] / (1.0f + expf(-g[e])) * u[e];
  Vec<T>::store(out + t * inter + (size_t)vi * N, o);
}

// The error words of the kernels that wait with a limit (defined beside those kernels).
int* gemm_tcgen05_error_address();
int* attention_error_address();
int* attention_tc_error_address();

__global__ void status_snapshot_kernel(const int* a, const int* b, const int* c, int* out) {
  pdl_wait();   // the kernels before this one on the stream have finished: what they recorded is seen
  if (threadIdx.x == 0) {
    out[0] = *a;
    out[1] = *b;
    out[2] = *c;
    out[3] = 1;   // says that the snapshot was written
    __threadfence_system();
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_status_snapshot(int32_t* out, int out_is_host, roost_stream_t stream) {
  ROOST_REQUIRE(out != nullptr, "status_snapshot: no destination");
  int* dst = out;
  if (out_is_host) {
    void* mapped = nullptr;
    if (cudaHostGetDevicePointer(&mapped, out, 0) != cudaSuccess || mapped == nullptr) {
      cudaGetLastError();
      return fail(ROOST_ERR_INVALID, "status_snapshot: the host destination is not page-locked memory the device can write");
    }
    dst = static_cast<int*>(mapped);
  }
  const int *a = gemm_tcgen05_error_address(), *b = attention_error_address(), *c = attention_tc_error_address();
  if (!a || !b || !c) return fail(ROOST_ERR_CUDA, "status_snapshot: an error word has no device address");
  cudaError_t e = launch_kernel(status_snapshot_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, a, b, c, dst);
  if (e != cudaSuccess) return fail(ROOST_ERR_CUDA, std::string("status_snapshot: ") + cudaGetErrorString(e));
  return ROOST_OK;
}

extern "C" int roost_abi_version(void) { return ROOST_ABI_VERSION; }
extern "C" void roost_set_pdl(int on) { g_pdl_enabled = on != 0; }
extern "C" const char* roost_last_error(void) { return g_last_error.c_str(); }

extern "C" int roost_embedding(const void* table, const int32_t* ids, void* out, int tokens, int hidden, int vocab,
                               int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0, "embedding: tokens, hidden and vocab must be positive");
  if (tokens == 0) return ROOST_OK;
  ROOST_DISPATCH_DTYPE(dtype, T,
                       launch_kernel(embedding_kernel<T>, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, (const T*)table, ids, (T*)out, hidden, vocab));
  return check_launch("embedding");
}

template <bool ADD>
static int launch_norm(const void* x, void* residual, const void* w, void* out, const int32_t* rows, int n_out,
                       int hidden, float eps, int dtype, int wdtype, roost_stream_t stream) {
  ROOST_REQUIRE(n_out >= 0 && hidden > 0, "rms_norm: rows and hidden must be positive");
  ROOST_REQUIRE(eps > 0.f, "rms_norm: eps must be positive");
  ROOST_REQUIRE(wdtype == ROOST_F32 || wdtype == ROOST_BF16, "rms_norm: weight dtype code is neither 0 nor 1");
  if (n_out == 0) return ROOST_OK;
  // rows that are whole 16-byte vectors and fit in registers take the vectorised kernel
  {
    const int vec = dtype == ROOST_F32 ? 4 : 8;
    const bool aligned = ((uintptr_t)x % 16 == 0) && ((uintptr_t)out % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
                         (!ADD || (uintptr_t)residual % 16 == 0);
    if (hidden % vec == 0 && aligned && (dtype == ROOST_F32 || dtype == ROOST_BF16)) {
      const int nvec = hidden / vec;
      int threads = ((nvec + 31) / 32) * 32;
      if (threads > 512) threads = 512;
      // many rows of bfloat16: four vectors a thread, so that a block waits less at its reduction and more rows are in
      // flight on an SM (float32 keeps one order of summation whatever the number of rows: its bits do not depend on the batch)
      if (dtype == ROOST_BF16 && n_out >= kNormWideRows && nvec >= 4 * 32) threads = (((nvec + 3) / 4 + 31) / 32) * 32;
      if (nvec <= threads * kMaxVec) {
        ROOST_DISPATCH_DTYPE(dtype, T, {
          auto kernel = n_out <= 64 ? rms_norm_vec_kernel<T, ADD, true> : rms_norm_vec_kernel<T, ADD, false>;
          launch_kernel(kernel, dim3(n_out), dim3(threads), 0, (cudaStream_t)stream, (const T*)x, (T*)residual, w, (T*)out, rows, hidden, eps,
                        wdtype);
        });
        return check_launch("rms_norm");
      }
    }
  }
  const size_t smem = ((size_t)hidden + 32) * sizeof(float);
  if (smem > 200 * 1024) return fail(ROOST_ERR_UNSUPPORTED, "rms_norm: a row of more than 51168 elements does not fit in shared memory");
  const int threads = hidden >= 1024 ? 512 : (hidden >= 256 ? 256 : 64);
  ROOST_DISPATCH_DTYPE(dtype, T, {
    auto kernel = rms_norm_kernel<T, ADD>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kernel, dim3(n_out), dim3(threads), smem, (cudaStream_t)stream, (const T*)x, (T*)residual, w, (T*)out, rows, hidden, eps,
                  wdtype);
  });
  return check_launch("rms_norm");
}

extern "C" int roost_rms_norm(const void* x, const void* w, void* out, const int32_t* rows, int n_out, int hidden,
                              float eps, int dtype, int wdtype, roost_stream_t stream) {
  return launch_norm<false>(x, nullptr, w, out, rows, n_out, hidden, eps, dtype, wdtype, stream);
}

extern "C" int roost_add_rms_norm(const void* x, void* residual, const void* w, void* out, const int32_t* rows,
                                  int n_out, int hidden, float eps, int dtype, int wdtype, roost_stream_t stream) {
  ROOST_REQUIRE(residual != nullptr, "add_rms_norm: residual is null");
  return launch_norm<true>(x, residual, w, out, rows, n_out, hidden, eps, dtype, wdtype, stream);
}

extern "C" int roost_silu_mul(const void* x, void* out, int tokens, int inter, int block, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && inter > 0, "silu_mul: tokens and inter must be positive");
  ROOST_REQUIRE(block >= 0 && (block == 0 || (inter % block == 0 && block % 8 == 0)),
                "silu_mul: the interleave block must divide inter and be a multiple of 8");
  if (tokens == 0) return ROOST_OK;
  {
    const int vec = dtype == ROOST_F32 ? 4 : 8;
    if (inter % vec == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0 && (dtype == ROOST_F32 || dtype == ROOST_BF16)) {
      const int nvec = inter / vec;
      dim3 grid(tokens, (nvec + 127) / 128);
      if (grid.y <= 65535) {
        ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(silu_mul_vec_kernel<T>, grid, dim3(128), 0, (cudaStream_t)stream, (const T*)x, (T*)out, inter, block));
        return check_launch("silu_mul");
      }
    }
  }
  if ((inter + 255) / 256 > 65535) return fail(ROOST_ERR_UNSUPPORTED, "silu_mul: inter beyond 16776960");
  dim3 grid(tokens, (inter + 255) / 256);
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(silu_mul_kernel<T>, grid, dim3(256), 0, (cudaStream_t)stream, (const T*)x, (T*)out, inter, block));
  return check_launch("silu_mul");
}

ROOST_TRACE_TU(elementwise)
