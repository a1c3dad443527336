// Streaming kernels for the per-irrep layers that follow a tensor product (gate, norms, RMS normalisation).
//
//   irrep_scale:  out[n, i, c] = x[n, i, c] * s(n, irrep(i), c)        s given per sample and channel (N, K, C),
//                                                                       shared (K, C) or per sample (N, K)
//   irrep_dot:    out[n, k, c] = sum_{i in irrep k} a[n, i, c] * b[n, i, c]
//
// Both are pure HBM streams over (N, D, C) features: one 128-bit load per operand and element group, the
// irrep of a component comes from a table in shared memory, no index loads from global memory.  The gate,
// the application of a normalisation and every gradient of these layers are instances of the two.
#include "common.cuh"

namespace eqt {
namespace {

constexpr int MAX_COMPONENTS = 1024;   // irreps.dim handled by the shared-memory irrep table

template <typename T, int V> struct Vec;
template <> struct Vec<float, 4> { using type = float4; };
template <> struct Vec<double, 2> { using type = double2; };
template <> struct Vec<float, 1> { using type = float; };
template <> struct Vec<double, 1> { using type = double; };

template <typename T, int V>
__device__ __forceinline__ void load(const T* p, T (&v)[V]) {
  const typename Vec<T, V>::type t = __ldg(reinterpret_cast<const typename Vec<T, V>::type*>(p));
  const T* q = reinterpret_cast<const T*>(&t);
#pragma unroll
  for (int i = 0; i < V; ++i) v[i] = q[i];
}
template <typename T, int V>
__device__ __forceinline__ void store(T* p, const T (&v)[V]) {
  typename Vec<T, V>::type t;
  T* q = reinterpret_cast<T*>(&t);
#pragma unroll
  for (int i = 0; i < V; ++i) q[i] = v[i];
  *reinterpret_cast<typename Vec<T, V>::type*>(p) = t;
}

// s_mode: 0 = s (N, K, C), 1 = s (K, C), 2 = s (N, K)
template <typename T, int V>
__global__ void __launch_bounds__(256) irrep_scale_kernel(const T* __restrict__ x, const T* __restrict__ s, T* __restrict__ out,
                                                          const int64_t* __restrict__ irrep_index, int64_t n, int d, int k,
                                                          int c, int s_mode) {
  __shared__ uint16_t kidx[MAX_COMPONENTS];
  for (int i = threadIdx.x; i < d; i += blockDim.x) kidx[i] = (uint16_t)__ldg(irrep_index + i);
  __syncthreads();
  const int cv = c / V;
  const int64_t per_sample = (int64_t)d * cv, total = n * per_sample;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = idx / per_sample;
    const int rem = (int)(idx - row * per_sample);
    const int i = rem / cv, c0 = (rem - i * cv) * V;
    const int kk = kidx[i];
    T xv[V], sv[V], ov[V];
    load<T, V>(x + (row * d + i) * c + c0, xv);
    if (s_mode == 2) {
      const T t = __ldg(s + row * k + kk);
#pragma unroll
      for (int q = 0; q < V; ++q) sv[q] = t;
    } else {
      load<T, V>(s + ((s_mode == 0 ? row * k : 0) + kk) * c + c0, sv);
    }
#pragma unroll
    for (int q = 0; q < V; ++q) ov[q] = xv[q] * sv[q];
    store<T, V>(out + (row * d + i) * c + c0, ov);
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(256) irrep_dot_kernel(const T* a, const T* b, T* __restrict__ out,
                                                        const int64_t* __restrict__ irrep_seg, int64_t n, int d, int k, int c) {
  __shared__ int seg[MAX_COMPONENTS + 1];
  for (int i = threadIdx.x; i <= k; i += blockDim.x) seg[i] = (int)__ldg(irrep_seg + i);
  __syncthreads();
  const int cv = c / V;
  const int64_t per_sample = (int64_t)k * cv, total = n * per_sample;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = idx / per_sample;
    const int rem = (int)(idx - row * per_sample);
    const int kk = rem / cv, c0 = (rem - kk * cv) * V;
    T acc[V];
#pragma unroll
    for (int q = 0; q < V; ++q) acc[q] = T(0);
    for (int i = seg[kk]; i < seg[kk + 1]; ++i) {
      T av[V], bv[V];
      load<T, V>(a + (row * d + i) * c + c0, av);
      if (a == b) {
#pragma unroll
        for (int q = 0; q < V; ++q) acc[q] = fma(av[q], av[q], acc[q]);
      } else {
        load<T, V>(b + (row * d + i) * c + c0, bv);
#pragma unroll
        for (int q = 0; q < V; ++q) acc[q] = fma(av[q], bv[q], acc[q]);
      }
    }
    store<T, V>(out + (row * k + kk) * c + c0, acc);
  }
}

template <typename T, int V>
int run_scale(const void* x, const void* s, void* out, const int64_t* index, int64_t n, int d, int k, int c, int mode,
              cudaStream_t st) {
  const int64_t work = n * d * (c / V);
  irrep_scale_kernel<T, V><<<flat_grid(work, 256, 148 * 16), 256, 0, st>>>(static_cast<const T*>(x), static_cast<const T*>(s),
                                                                            static_cast<T*>(out), index, n, d, k, c, mode);
  return check_launch("irrep_scale_kernel");
}
template <typename T, int V>
int run_dot(const void* a, const void* b, void* out, const int64_t* seg, int64_t n, int d, int k, int c, cudaStream_t st) {
  const int64_t work = n * k * (c / V);
  irrep_dot_kernel<T, V><<<flat_grid(work, 256, 148 * 16), 256, 0, st>>>(static_cast<const T*>(a), static_cast<const T*>(b),
                                                                          static_cast<T*>(out), seg, n, d, k, c);
  return check_launch("irrep_dot_kernel");
}

int check_sizes(int64_t n, int d, int k, int c, int dtype) {
  if (n < 0 || d <= 0 || k <= 0 || c <= 0) return fail(EQT_ERR_BAD_ARGUMENT, "bad sizes");
  if (d > MAX_COMPONENTS || k > d) return fail(EQT_ERR_UNSUPPORTED, "at most %d components, num_irreps <= components", MAX_COMPONENTS);
  if (dtype != EQT_F32 && dtype != EQT_F64) return fail(EQT_ERR_UNSUPPORTED, "float32 or float64 only");
  return EQT_OK;
}
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace eqt

extern "C" int eqt_irrep_scale(const void* x, const void* s, void* out, const int64_t* irrep_index, int64_t n, int32_t d,
                               int32_t k, int32_t c, int32_t s_mode, int32_t dtype, void* stream) {
  using namespace eqt;
  if (int rc = check_sizes(n, d, k, c, dtype)) return rc;
  if (s_mode < 0 || s_mode > 2) return fail(EQT_ERR_BAD_ARGUMENT, "s_mode must be 0, 1 or 2");
  if (n == 0) return EQT_OK;
  if (!x || !s || !out || !irrep_index) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec_ok = aligned16(x) && aligned16(out) && (s_mode == 2 || aligned16(s));
  if (dtype == EQT_F32) {
    if (c % 4 == 0 && vec_ok) return run_scale<float, 4>(x, s, out, irrep_index, n, d, k, c, s_mode, st);
    return run_scale<float, 1>(x, s, out, irrep_index, n, d, k, c, s_mode, st);
  }
  if (c % 2 == 0 && vec_ok) return run_scale<double, 2>(x, s, out, irrep_index, n, d, k, c, s_mode, st);
  return run_scale<double, 1>(x, s, out, irrep_index, n, d, k, c, s_mode, st);
}

extern "C" int eqt_irrep_dot(const void* a, const void* b, void* out, const int64_t* irrep_seg, int64_t n, int32_t d,
                             int32_t k, int32_t c, int32_t dtype, void* stream) {
  using namespace eqt;
  if (int rc = check_sizes(n, d, k, c, dtype)) return rc;
  if (n == 0) return EQT_OK;
  if (!a || !b || !out || !irrep_seg) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec_ok = aligned16(a) && aligned16(b) && aligned16(out);
  if (dtype == EQT_F32) {
    if (c % 4 == 0 && vec_ok) return run_dot<float, 4>(a, b, out, irrep_seg, n, d, k, c, st);
    return run_dot<float, 1>(a, b, out, irrep_seg, n, d, k, c, st);
  }
  if (c % 2 == 0 && vec_ok) return run_dot<double, 2>(a, b, out, irrep_seg, n, d, k, c, st);
  return run_dot<double, 1>(a, b, out, irrep_seg, n, d, k, c, st);
}
