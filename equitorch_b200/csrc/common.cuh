// Shared helpers for the eqt_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdio>

#include "../../include/eqt_b200.h"

namespace eqt {

// ---- error reporting ------------------------------------------------------------------
char* error_buffer();                       // thread-local, 512 bytes
int fail(int code, const char* fmt, ...);   // formats into error_buffer(), returns code
extern std::atomic<int64_t> g_launches;

inline int check_launch(const char* what) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(EQT_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return EQT_OK;
}

// ---- storage <-> arithmetic types --------------------------------------------------------
template <typename T> struct Acc { using type = float; };
template <> struct Acc<double> { using type = double; };

template <typename T> __device__ __forceinline__ typename Acc<T>::type ld(const T* p) { return __ldg(p); }
template <> __device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <typename T, typename A> __device__ __forceinline__ void st(T* p, A v) { *p = static_cast<T>(v); }
template <> __device__ __forceinline__ void st<__nv_bfloat16, float>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

__host__ __device__ inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Number of SMs of the current device (queried once per device ordinal).
int sm_count();

// Grid size for a flat 1-D launch: enough blocks for `work` items, capped at `blocks_per_sm` blocks per
// SM of the current device so that one wave of a grid-stride loop fills the GPU a few times over.
inline unsigned flat_grid(int64_t work, int threads, int blocks_per_sm = 32) {
  int64_t b = ceil_div(work, threads);
  const int64_t max_blocks = (int64_t)sm_count() * blocks_per_sm;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return static_cast<unsigned>(b);
}

}  // namespace eqt
