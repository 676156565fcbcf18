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

// ---------------------------------------------------------------------------------------------- embedding
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int32_t* __restrict__ ids, T* __restrict__ out,
                                 int hidden, int vocab) {
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
__global__ void silu_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int inter) {
  const size_t t = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= inter) return;
  const float g = to_float(x[t * 2 * inter + i]);
  const float u = to_float(x[t * 2 * inter + inter + i]);
  out[t * inter + i] = from_float<T>(g / (1.0f + expf(-g)) * u);
}

}  // namespace roost

using namespace roost;

extern "C" int roost_abi_version(void) { return ROOST_ABI_VERSION; }
extern "C" const char* roost_last_error(void) { return g_last_error.c_str(); }

extern "C" int roost_embedding(const void* table, const int32_t* ids, void* out, int tokens, int hidden, int vocab,
                               int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0, "embedding: tokens, hidden and vocab must be positive");
  if (tokens == 0) return ROOST_OK;
  ROOST_DISPATCH_DTYPE(dtype, T,
                       embedding_kernel<T><<<tokens, 256, 0, (cudaStream_t)stream>>>((const T*)table, ids, (T*)out, hidden, vocab));
  return check_launch("embedding");
}

template <bool ADD>
static int launch_norm(const void* x, void* residual, const void* w, void* out, const int32_t* rows, int n_out,
                       int hidden, float eps, int dtype, int wdtype, roost_stream_t stream) {
  ROOST_REQUIRE(n_out >= 0 && hidden > 0, "rms_norm: rows and hidden must be positive");
  ROOST_REQUIRE(eps > 0.f, "rms_norm: eps must be positive");
  ROOST_REQUIRE(wdtype == ROOST_F32 || wdtype == ROOST_BF16, "rms_norm: weight dtype code is neither 0 nor 1");
  if (n_out == 0) return ROOST_OK;
  const size_t smem = ((size_t)hidden + 32) * sizeof(float);
  if (smem > 200 * 1024) return fail(ROOST_ERR_UNSUPPORTED, "rms_norm: a row of more than 51168 elements does not fit in shared memory");
  const int threads = hidden >= 1024 ? 512 : (hidden >= 256 ? 256 : 64);
  ROOST_DISPATCH_DTYPE(dtype, T, {
    auto kernel = rms_norm_kernel<T, ADD>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kernel<<<n_out, threads, smem, (cudaStream_t)stream>>>((const T*)x, (T*)residual, w, (T*)out, rows, hidden, eps, wdtype);
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

extern "C" int roost_silu_mul(const void* x, void* out, int tokens, int inter, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && inter > 0, "silu_mul: tokens and inter must be positive");
  if (tokens == 0) return ROOST_OK;
  if ((inter + 255) / 256 > 65535) return fail(ROOST_ERR_UNSUPPORTED, "silu_mul: inter beyond 16776960");
  dim3 grid(tokens, (inter + 255) / 256);
  ROOST_DISPATCH_DTYPE(dtype, T, silu_mul_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>((const T*)x, (T*)out, inter));
  return check_launch("silu_mul");
}
