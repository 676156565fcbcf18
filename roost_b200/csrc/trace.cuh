// Development instrumentation, included by common.cuh only in builds with -DROOST_TRACE (the product build never sees
// this file): thread 0 of every block appends (tag * 4 + phase, block, nanoseconds) to a buffer bound by
// roost_trace_bind_<file>; phase 0 is the block's start, 1 the return of pdl_wait, 2 its end.
#pragma once

namespace roost {

static __device__ unsigned long long* g_trace;  // [0]: number of records; then two words a record
__device__ __forceinline__ void trace_point(int tag, int phase) {
  if (tag && threadIdx.x == 0 && g_trace) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    const unsigned long long i = atomicAdd(g_trace, 1ULL);
    if (i < (1ULL << 20)) {
      g_trace[1 + 2 * i] = ((unsigned long long)(tag * 4 + phase) << 32) | (blockIdx.y << 16) | blockIdx.x;
      g_trace[2 + 2 * i] = t;
    }
  }
}
// Events a thread timed itself (trace_now) and kept in registers, written out when its work is done: n records of
// (code, first value + index, nanoseconds). The caller picks which blocks and threads record.
__device__ __forceinline__ unsigned long long trace_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}
__device__ __forceinline__ void trace_flush(int code, int first, const unsigned long long* times, int n) {
  if (g_trace && n > 0) {
    const unsigned long long i0 = atomicAdd(g_trace, (unsigned long long)n);
    for (int k = 0; k < n; ++k) {
      const unsigned long long i = i0 + k;
      if (i < (1ULL << 20)) {
        g_trace[1 + 2 * i] = ((unsigned long long)code << 32) | (unsigned int)(first + k);
        g_trace[2 + 2 * i] = times[k];
      }
    }
  }
}
#define ROOST_TRACE_TU(name) \
  extern "C" void roost_trace_bind_##name(void* p) { cudaMemcpyToSymbol(roost::g_trace, &p, sizeof(p)); }

}  // namespace roost
