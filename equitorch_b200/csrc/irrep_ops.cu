// Streaming kernels for the per-irrep layers that follow a tensor product (gate, norms, RMS normalisation).
//
//   irrep_scale:  out[n, i, c] = x[n, i, c] * s(n, irrep(i), c)        s given per sample and channel (N, K, C),
//                                                                       shared (K, C) or per sample (N, K)
//   irrep_dot:    out[n, k, c] = sum_{i in irrep k} a[n, i, c] * b[n, i, c]
//
// Both are pure HBM streams over (N, D, C) features: one 128-bit load per operand and element group, the
// irrep of a component comes from a table in shared memory, no index loads from global memory.  The gate,
// the application of a normalisation and every gradient of these layers are instances of the two.
#include <algorithm>

#include "common.cuh"

namespace eqt {
namespace {

constexpr int MAX_COMPONENTS = 1024;   // irreps.dim handled by the shared-memory irrep table

template <typename T, int V> struct Vec;
template <> struct Vec<float, 4> { using type = float4; };
template <> struct Vec<double, 2> { using type = double2; };
template <> struct Vec<float, 1> { using type = float; };
template <> struct Vec<double, 1> { using type = double; };
template <> struct Vec<__nv_bfloat16, 8> { using type = uint4; };
template <> struct Vec<__nv_bfloat16, 1> { using type = __nv_bfloat16; };

// V storage elements of type T <-> V values of the arithmetic type (float for bfloat16 storage)
template <typename T, int V>
__device__ __forceinline__ void load(const T* p, typename Acc<T>::type (&v)[V]) {
  const typename Vec<T, V>::type t = __ldg(reinterpret_cast<const typename Vec<T, V>::type*>(p));
  const T* q = reinterpret_cast<const T*>(&t);
#pragma unroll
  for (int i = 0; i < V; ++i) v[i] = static_cast<typename Acc<T>::type>(q[i]);
}
template <typename T, int V>
__device__ __forceinline__ void store(T* p, const typename Acc<T>::type (&v)[V]) {
  typename Vec<T, V>::type t;
  T* q = reinterpret_cast<T*>(&t);
#pragma unroll
  for (int i = 0; i < V; ++i) q[i] = static_cast<T>(v[i]);
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
    typename Acc<T>::type xv[V], sv[V], ov[V];
    load<T, V>(x + (row * d + i) * c + c0, xv);
    if (s_mode == 2) {
      const typename Acc<T>::type t = ld(s + row * k + kk);
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
    using A = typename Acc<T>::type;
    A acc[V];
#pragma unroll
    for (int q = 0; q < V; ++q) acc[q] = A(0);
    for (int i = seg[kk]; i < seg[kk + 1]; ++i) {
      A av[V], bv[V];
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
  irrep_scale_kernel<T, V><<<flat_grid(work, 256, 16), 256, 0, st>>>(static_cast<const T*>(x), static_cast<const T*>(s),
                                                                            static_cast<T*>(out), index, n, d, k, c, mode);
  return check_launch("irrep_scale_kernel");
}
template <typename T, int V>
int run_dot(const void* a, const void* b, void* out, const int64_t* seg, int64_t n, int d, int k, int c, cudaStream_t st) {
  const int64_t work = n * k * (c / V);
  irrep_dot_kernel<T, V><<<flat_grid(work, 256, 16), 256, 0, st>>>(static_cast<const T*>(a), static_cast<const T*>(b),
                                                                          static_cast<T*>(out), seg, n, d, k, c);
  return check_launch("irrep_dot_kernel");
}

int check_sizes(int64_t n, int d, int k, int c, int dtype) {
  if (n < 0 || d <= 0 || k <= 0 || c <= 0) return fail(EQT_ERR_BAD_ARGUMENT, "bad sizes");
  if (d > MAX_COMPONENTS || k > d) return fail(EQT_ERR_UNSUPPORTED, "at most %d components, num_irreps <= components", MAX_COMPONENTS);
  if (dtype != EQT_F32 && dtype != EQT_F64 && dtype != EQT_BF16) return fail(EQT_ERR_UNSUPPORTED, "float32, float64 or bfloat16 only");
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
  if (dtype == EQT_BF16) {   // bfloat16 storage, float32 arithmetic
    if (c % 8 == 0 && vec_ok) return run_scale<__nv_bfloat16, 8>(x, s, out, irrep_index, n, d, k, c, s_mode, st);
    return run_scale<__nv_bfloat16, 1>(x, s, out, irrep_index, n, d, k, c, s_mode, st);
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
  if (dtype == EQT_BF16) {
    if (c % 8 == 0 && vec_ok) return run_dot<__nv_bfloat16, 8>(a, b, out, irrep_seg, n, d, k, c, st);
    return run_dot<__nv_bfloat16, 1>(a, b, out, irrep_seg, n, d, k, c, st);
  }
  if (c % 2 == 0 && vec_ok) return run_dot<double, 2>(a, b, out, irrep_seg, n, d, k, c, st);
  return run_dot<double, 1>(a, b, out, irrep_seg, n, d, k, c, st);
}

// ------------------------------------------------------------------------------------------------------
// Fused LayerRMSNorm: one warp per sample.  The components of an irrep are a contiguous run of dim_k * C
// floats, so the warp sums the squares of the run, turns the sum into 1/sigma and rescales the run (second
// read from L1): one HBM read and one write per element instead of four passes.  The backward pass is fused
// the same way; the gradient of the weight is accumulated per lane over the warp's samples (a lane always
// meets the same channels because C / V divides 32) and written as one partial per warp, summed by the caller
// in a fixed order.
// ------------------------------------------------------------------------------------------------------
namespace eqt {
namespace {

constexpr int LRN_MAX_IRREPS = 16;

template <typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <typename T> __device__ __forceinline__ T rsqrt_t(T v);
template <> __device__ __forceinline__ float rsqrt_t<float>(float v) { return 1.0f / sqrtf(v); }
template <> __device__ __forceinline__ double rsqrt_t<double>(double v) { return 1.0 / sqrt(v); }

template <typename T, int V>
__global__ void __launch_bounds__(256) layer_rms_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ out,
                                                            T* __restrict__ rsigma, const int64_t* __restrict__ irrep_seg,
                                                            int64_t n, int d, int k, int c, int scaled, T eps) {
  __shared__ int seg[LRN_MAX_IRREPS + 1];
  for (int i = threadIdx.x; i <= k; i += blockDim.x) seg[i] = (int)__ldg(irrep_seg + i);
  __syncthreads();
  const int lane = threadIdx.x & 31, cv = c / V;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = warp; row < n; row += warps) {
    for (int kk = 0; kk < k; ++kk) {
      const int dim = seg[kk + 1] - seg[kk], vecs = dim * cv;
      const T* xr = x + (row * d + seg[kk]) * c;
      T* orow = out + (row * d + seg[kk]) * c;
      T sum = T(0);
      for (int j = lane; j < vecs; j += 32) {
        T v[V];
        load<T, V>(xr + j * V, v);
#pragma unroll
        for (int q = 0; q < V; ++q) sum = fma(v[q], v[q], sum);
      }
      sum = warp_sum(sum);
      const T stat = sum / T(c) * (scaled ? T(1) / T(dim) : T(1));
      const T r = rsqrt_t<T>(stat + eps);
      if (lane == 0) rsigma[row * k + kk] = r;
      for (int j = lane; j < vecs; j += 32) {
        T v[V], wv[V];
        load<T, V>(xr + j * V, v);
        if (w) {
          load<T, V>(w + kk * c + (j % cv) * V, wv);
#pragma unroll
          for (int q = 0; q < V; ++q) v[q] = v[q] * r * wv[q];
        } else {
#pragma unroll
          for (int q = 0; q < V; ++q) v[q] = v[q] * r;
        }
        store<T, V>(orow + j * V, v);
      }
    }
  }
}

// gx = r w go - x r^3 t / (C [dim]),  t = sum over the irrep block of go w x;  gw partial per warp
template <typename T, int V>
__global__ void __launch_bounds__(256) layer_rms_bwd_kernel(const T* __restrict__ x, const T* __restrict__ go, const T* __restrict__ w,
                                                            const T* __restrict__ rsigma, T* __restrict__ gx, T* __restrict__ gw_partial,
                                                            const int64_t* __restrict__ irrep_seg, int64_t n, int d, int k, int c,
                                                            int scaled) {
  __shared__ int seg[LRN_MAX_IRREPS + 1];
  for (int i = threadIdx.x; i <= k; i += blockDim.x) seg[i] = (int)__ldg(irrep_seg + i);
  __syncthreads();
  const int lane = threadIdx.x & 31, cv = c / V;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  T gwa[LRN_MAX_IRREPS][V];
#pragma unroll
  for (int kk = 0; kk < LRN_MAX_IRREPS; ++kk)
#pragma unroll
    for (int q = 0; q < V; ++q) gwa[kk][q] = T(0);
  const int cslot = lane % cv;   // the channel group this lane meets in every run (cv divides 32)
  for (int64_t row = warp; row < n; row += warps) {
#pragma unroll
    for (int kk = 0; kk < LRN_MAX_IRREPS; ++kk) {
      if (kk >= k) break;
      const int dim = seg[kk + 1] - seg[kk], vecs = dim * cv;
      const int64_t off = (row * d + seg[kk]) * c;
      const T r = __ldg(rsigma + row * k + kk);
      T wv[V];
      if (w) load<T, V>(w + kk * c + cslot * V, wv);
      else {
#pragma unroll
        for (int q = 0; q < V; ++q) wv[q] = T(1);
      }
      T t = T(0);
      for (int j = lane; j < vecs; j += 32) {
        T xv[V], gv[V];
        load<T, V>(x + off + j * V, xv);
        load<T, V>(go + off + j * V, gv);
#pragma unroll
        for (int q = 0; q < V; ++q) {
          const T gxv = gv[q] * xv[q];
          t = fma(gxv, wv[q], t);
          gwa[kk][q] = fma(gxv, r, gwa[kk][q]);
        }
      }
      t = warp_sum(t);
      const T coef = t * r * r * r / (T(c) * (scaled ? T(dim) : T(1)));
      for (int j = lane; j < vecs; j += 32) {
        T xv[V], gv[V];
        load<T, V>(x + off + j * V, xv);
        load<T, V>(go + off + j * V, gv);
#pragma unroll
        for (int q = 0; q < V; ++q) gv[q] = r * wv[q] * gv[q] - xv[q] * coef;
        store<T, V>(gx + off + j * V, gv);
      }
    }
  }
  if (gw_partial) {
    // lanes with the same channel group (lane, lane + cv, ...) hold partial sums of the same weights: fold them
#pragma unroll
    for (int kk = 0; kk < LRN_MAX_IRREPS; ++kk) {
      if (kk >= k) break;
#pragma unroll
      for (int q = 0; q < V; ++q) {
        T v = gwa[kk][q];
        for (int o = 16; o >= cv; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        gwa[kk][q] = v;
      }
      if (lane < cv && warp < warps) store<T, V>(gw_partial + (warp * k + kk) * c + lane * V, gwa[kk]);
    }
  }
}

template <typename T> struct LrnVec;
template <> struct LrnVec<float> { static constexpr int V = 4; };
template <> struct LrnVec<double> { static constexpr int V = 2; };

int layer_rms_grid(int64_t n) {
  // eight warps per CTA, a few CTAs per SM; each warp walks samples with stride `warps`
  return (int)std::max<int64_t>(1, std::min<int64_t>((n + 7) / 8, (int64_t)sm_count() * 8));
}

bool layer_rms_ok(int d, int k, int c, int v) {
  return k <= LRN_MAX_IRREPS && d <= MAX_COMPONENTS && c % v == 0 && 32 % (c / v) == 0;
}

}  // namespace
}  // namespace eqt

extern "C" int eqt_layer_rms_num_partials(int64_t n) { return eqt::layer_rms_grid(n) * 8; }

extern "C" int eqt_layer_rms_forward(const void* x, const void* weight, void* out, void* rsigma, const int64_t* irrep_seg,
                                     int64_t n, int32_t d, int32_t k, int32_t c, int32_t scaled, double eps, int32_t dtype,
                                     void* stream) {
  using namespace eqt;
  if (int rc = check_sizes(n, d, k, c, dtype)) return rc;
  if (n == 0) return EQT_OK;
  if (!x || !out || !rsigma || !irrep_seg) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  const int v = dtype == EQT_F32 ? 4 : 2;
  if (!layer_rms_ok(d, k, c, v) || !aligned16(x) || !aligned16(out) || (weight && !aligned16(weight)))
    return fail(EQT_ERR_UNSUPPORTED, "fused LayerRMSNorm needs <= %d irreps, C / %d dividing 32 and 16-byte aligned tensors",
                LRN_MAX_IRREPS, v);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = layer_rms_grid(n);
  if (dtype == EQT_F32)
    layer_rms_fwd_kernel<float, 4><<<grid, 256, 0, st>>>(static_cast<const float*>(x), static_cast<const float*>(weight),
                                                         static_cast<float*>(out), static_cast<float*>(rsigma), irrep_seg, n, d, k,
                                                         c, scaled, (float)eps);
  else
    layer_rms_fwd_kernel<double, 2><<<grid, 256, 0, st>>>(static_cast<const double*>(x), static_cast<const double*>(weight),
                                                          static_cast<double*>(out), static_cast<double*>(rsigma), irrep_seg, n, d,
                                                          k, c, scaled, eps);
  return check_launch("layer_rms_fwd_kernel");
}

extern "C" int eqt_layer_rms_backward(const void* x, const void* grad_out, const void* weight, const void* rsigma, void* grad_x,
                                      void* grad_weight_partial, const int64_t* irrep_seg, int64_t n, int32_t d, int32_t k,
                                      int32_t c, int32_t scaled, int32_t dtype, void* stream) {
  using namespace eqt;
  if (int rc = check_sizes(n, d, k, c, dtype)) return rc;
  if (n == 0) return EQT_OK;
  if (!x || !grad_out || !rsigma || !grad_x || !irrep_seg) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  const int v = dtype == EQT_F32 ? 4 : 2;
  if (!layer_rms_ok(d, k, c, v) || !aligned16(x) || !aligned16(grad_out) || !aligned16(grad_x) || (weight && !aligned16(weight)) ||
      (grad_weight_partial && !aligned16(grad_weight_partial)))
    return fail(EQT_ERR_UNSUPPORTED, "fused LayerRMSNorm needs <= %d irreps, C / %d dividing 32 and 16-byte aligned tensors",
                LRN_MAX_IRREPS, v);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = layer_rms_grid(n);
  if (dtype == EQT_F32)
    layer_rms_bwd_kernel<float, 4><<<grid, 256, 0, st>>>(static_cast<const float*>(x), static_cast<const float*>(grad_out),
                                                         static_cast<const float*>(weight), static_cast<const float*>(rsigma),
                                                         static_cast<float*>(grad_x), static_cast<float*>(grad_weight_partial),
                                                         irrep_seg, n, d, k, c, scaled);
  else
    layer_rms_bwd_kernel<double, 2><<<grid, 256, 0, st>>>(static_cast<const double*>(x), static_cast<const double*>(grad_out),
                                                          static_cast<const double*>(weight), static_cast<const double*>(rsigma),
                                                          static_cast<double*>(grad_x), static_cast<double*>(grad_weight_partial),
                                                          irrep_seg, n, d, k, c, scaled);
  return check_launch("layer_rms_bwd_kernel");
}
