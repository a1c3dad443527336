// Spherical harmonics (table-driven degree recurrence, forward and reverse mode) and the
// row gather / CSR segment-sum that surround a tensor-product layer in a graph network.
#include <algorithm>

#include "common.cuh"

namespace eqt {
namespace {

#include "generated/sh_specs.inc"

struct ShTab {
  const int32_t* ptr;
  const int32_t* m_out;
  const int32_t* m_in;
  const int32_t* axis;
  const double* coef;
  int l_max;
};

// One thread per point.  All (l_max+1)^2 values of a point live in one shared-memory column
// (component-major, thread-minor => conflict free); the block then writes its contiguous
// slab of the output with coalesced stores.
template <typename T>
__global__ void sh_forward_kernel(const T* __restrict__ xyz, T* __restrict__ out, int64_t n, ShTab tab,
                                  int normalize, typename Acc<T>::type out_scale) {
  using A = typename Acc<T>::type;
  extern __shared__ unsigned char smem_raw[];
  A* col = reinterpret_cast<A*>(smem_raw);
  const int K = (tab.l_max + 1) * (tab.l_max + 1);
  const int B = blockDim.x, tid = threadIdx.x;
  for (int64_t base = (int64_t)blockIdx.x * B; base < n; base += (int64_t)gridDim.x * B) {
    const int64_t pt = base + tid;
    if (pt < n) {
      A r[3] = {ld(xyz + pt * 3), ld(xyz + pt * 3 + 1), ld(xyz + pt * 3 + 2)};
      if (normalize) {
        const A inv = A(1) / max(sqrt(r[0] * r[0] + r[1] * r[1] + r[2] * r[2]), A(1e-12));
        r[0] *= inv; r[1] *= inv; r[2] *= inv;
      }
      col[tid] = A(1);
      for (int l = 1; l <= tab.l_max; ++l) {
        A* cur = col + (l * l) * B + tid;
        const A* prev = col + ((l - 1) * (l - 1)) * B + tid;
        for (int m = 0; m < 2 * l + 1; ++m) cur[m * B] = A(0);
        for (int e = tab.ptr[l]; e < tab.ptr[l + 1]; ++e)
          cur[tab.m_out[e] * B] += static_cast<A>(tab.coef[e]) * r[tab.axis[e]] * prev[tab.m_in[e] * B];
      }
    }
    __syncthreads();
    const int64_t rows = min((int64_t)B, n - base);
    for (int64_t q = tid; q < rows * K; q += B) {
      const int th = q / K, comp = q % K;
      st(out + base * K + q, col[comp * B + th] * out_scale);
    }
    __syncthreads();
  }
}

// Reverse mode through forward-mode columns: alongside Y the three partial derivatives
// dY/dx, dY/dy, dY/dz of the previous and the current degree are kept in shared memory
// (8 columns of 2 l_max + 1 entries per thread), and the cotangent is contracted degree by
// degree, so nothing of size (l_max+1)^2 is stored.
template <typename T>
__global__ void sh_backward_kernel(const T* __restrict__ xyz, const T* __restrict__ gout, T* __restrict__ gxyz,
                                   int64_t n, ShTab tab, int normalize, typename Acc<T>::type out_scale) {
  using A = typename Acc<T>::type;
  extern __shared__ unsigned char smem_raw[];
  A* sm = reinterpret_cast<A*>(smem_raw);
  const int W = 2 * tab.l_max + 1, K = (tab.l_max + 1) * (tab.l_max + 1);
  const int B = blockDim.x, tid = threadIdx.x;
  // layout: [buffer 0/1][quantity 0..3 = Y, dx, dy, dz][component][thread]
  auto at = [&](int buf, int q, int m) -> A& { return sm[((buf * 4 + q) * W + m) * B + tid]; };
  for (int64_t pt = (int64_t)blockIdx.x * B + tid; pt < n; pt += (int64_t)gridDim.x * B) {
    A u[3] = {ld(xyz + pt * 3), ld(xyz + pt * 3 + 1), ld(xyz + pt * 3 + 2)};
    A r[3] = {u[0], u[1], u[2]};
    A norm = A(1);
    if (normalize) {
      norm = max(sqrt(u[0] * u[0] + u[1] * u[1] + u[2] * u[2]), A(1e-12));
      r[0] /= norm; r[1] /= norm; r[2] /= norm;
    }
    A g[3] = {0, 0, 0};
    at(0, 0, 0) = A(1);
    at(0, 1, 0) = at(0, 2, 0) = at(0, 3, 0) = A(0);
    const T* go = gout + pt * K;
    for (int l = 1; l <= tab.l_max; ++l) {
      const int cb = l & 1, pb = cb ^ 1;
      for (int m = 0; m < 2 * l + 1; ++m)
        for (int q = 0; q < 4; ++q) at(cb, q, m) = A(0);
      for (int e = tab.ptr[l]; e < tab.ptr[l + 1]; ++e) {
        const int mo = tab.m_out[e], mi = tab.m_in[e], ax = tab.axis[e];
        const A c = static_cast<A>(tab.coef[e]);
        const A yp = at(pb, 0, mi);
        at(cb, 0, mo) += c * r[ax] * yp;
        at(cb, 1, mo) += c * (r[ax] * at(pb, 1, mi) + (ax == 0 ? yp : A(0)));
        at(cb, 2, mo) += c * (r[ax] * at(pb, 2, mi) + (ax == 1 ? yp : A(0)));
        at(cb, 3, mo) += c * (r[ax] * at(pb, 3, mi) + (ax == 2 ? yp : A(0)));
      }
      for (int m = 0; m < 2 * l + 1; ++m) {
        const A w = ld(go + l * l + m);
        g[0] += w * at(cb, 1, m);
        g[1] += w * at(cb, 2, m);
        g[2] += w * at(cb, 3, m);
      }
    }
    g[0] *= out_scale; g[1] *= out_scale; g[2] *= out_scale;
    if (normalize) {
      // v = u / max(|u|, eps):  dv = (I - v v^T) / |u| above eps, I / eps below
      const A un = sqrt(u[0] * u[0] + u[1] * u[1] + u[2] * u[2]);
      if (un > A(1e-12)) {
        const A dot = g[0] * r[0] + g[1] * r[1] + g[2] * r[2];
        g[0] = (g[0] - r[0] * dot) / norm; g[1] = (g[1] - r[1] * dot) / norm; g[2] = (g[2] - r[2] * dot) / norm;
      } else {
        g[0] /= norm; g[1] /= norm; g[2] /= norm;
      }
    }
    st(gxyz + pt * 3, g[0]); st(gxyz + pt * 3 + 1, g[1]); st(gxyz + pt * 3 + 2, g[2]);
  }
}

template <typename Kern>
int configure_smem(Kern kern, size_t bytes) {
  if (bytes > 48 * 1024) {
    if (bytes > 227 * 1024) return fail(EQT_ERR_UNSUPPORTED, "l_max needs %zu bytes of shared memory", bytes);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return fail(EQT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  }
  return EQT_OK;
}

// Small l_max: the recurrence as straight-line code on registers (generated/sh_specs.inc).  The forward kernel
// still goes through a shared-memory transpose so that a block writes its slab of the output contiguously.
template <typename T, int LMAX>
__global__ void __launch_bounds__(256) sh_forward_unrolled_kernel(const T* __restrict__ xyz, T* __restrict__ out, int64_t n,
                                                                  int normalize, typename Acc<T>::type out_scale) {
  using A = typename Acc<T>::type;
  using U = ShUnrolled<A, LMAX>;
  constexpr int K = U::K;
  extern __shared__ unsigned char smem_raw[];
  A* col = reinterpret_cast<A*>(smem_raw);
  const int B = blockDim.x, tid = threadIdx.x;
  for (int64_t base = (int64_t)blockIdx.x * B; base < n; base += (int64_t)gridDim.x * B) {
    const int64_t pt = base + tid;
    if (pt < n) {
      A r[3] = {ld(xyz + pt * 3), ld(xyz + pt * 3 + 1), ld(xyz + pt * 3 + 2)};
      if (normalize) {
        const A inv = A(1) / max(sqrt(r[0] * r[0] + r[1] * r[1] + r[2] * r[2]), A(1e-12));
        r[0] *= inv; r[1] *= inv; r[2] *= inv;
      }
      A y[K];
      U::forward(r, y);
#pragma unroll
      for (int k = 0; k < K; ++k) col[k * B + tid] = y[k] * out_scale;
    }
    __syncthreads();
    const int64_t rows = min((int64_t)B, n - base);
    for (int64_t q = tid; q < rows * K; q += B) {
      const int th = q / K, comp = q % K;
      st(out + base * K + q, col[comp * B + th]);
    }
    __syncthreads();
  }
}

template <typename T, int LMAX>
__global__ void __launch_bounds__(256) sh_backward_unrolled_kernel(const T* __restrict__ xyz, const T* __restrict__ gout,
                                                                   T* __restrict__ gxyz, int64_t n, int normalize,
                                                                   typename Acc<T>::type out_scale) {
  using A = typename Acc<T>::type;
  using U = ShUnrolled<A, LMAX>;
  constexpr int K = U::K;
  for (int64_t pt = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; pt < n; pt += (int64_t)gridDim.x * blockDim.x) {
    A u[3] = {ld(xyz + pt * 3), ld(xyz + pt * 3 + 1), ld(xyz + pt * 3 + 2)};
    A r[3] = {u[0], u[1], u[2]};
    A norm = A(1);
    if (normalize) {
      norm = max(sqrt(u[0] * u[0] + u[1] * u[1] + u[2] * u[2]), A(1e-12));
      r[0] /= norm; r[1] /= norm; r[2] /= norm;
    }
    A go[K], g[3];
#pragma unroll
    for (int k = 0; k < K; ++k) go[k] = ld(gout + pt * K + k);
    U::backward(r, go, g);
    g[0] *= out_scale; g[1] *= out_scale; g[2] *= out_scale;
    if (normalize) {
      // v = u / max(|u|, eps):  dv = (I - v v^T) / |u| above eps, I / eps below
      const A un = sqrt(u[0] * u[0] + u[1] * u[1] + u[2] * u[2]);
      if (un > A(1e-12)) {
        const A dot = g[0] * r[0] + g[1] * r[1] + g[2] * r[2];
        g[0] = (g[0] - r[0] * dot) / norm; g[1] = (g[1] - r[1] * dot) / norm; g[2] = (g[2] - r[2] * dot) / norm;
      } else {
        g[0] /= norm; g[1] /= norm; g[2] /= norm;
      }
    }
    st(gxyz + pt * 3, g[0]); st(gxyz + pt * 3 + 1, g[1]); st(gxyz + pt * 3 + 2, g[2]);
  }
}

template <typename T, int LMAX>
int sh_launch_unrolled(bool backward, const void* xyz, const void* gout, void* out, int64_t n, int normalize, double out_scale,
                       cudaStream_t s) {
  using A = typename Acc<T>::type;
  constexpr int K = (LMAX + 1) * (LMAX + 1);
  const unsigned grid = flat_grid(n, 256, 8);
  if (backward) {
    sh_backward_unrolled_kernel<T, LMAX><<<grid, 256, 0, s>>>(static_cast<const T*>(xyz), static_cast<const T*>(gout),
                                                              static_cast<T*>(out), n, normalize, (A)out_scale);
    return check_launch("sh_backward_unrolled_kernel");
  }
  if (int rc = configure_smem(sh_forward_unrolled_kernel<T, LMAX>, sizeof(A) * K * 256)) return rc;
  sh_forward_unrolled_kernel<T, LMAX><<<grid, 256, sizeof(A) * K * 256, s>>>(static_cast<const T*>(xyz), static_cast<T*>(out), n,
                                                                             normalize, (A)out_scale);
  return check_launch("sh_forward_unrolled_kernel");
}

template <typename T>
__global__ void __launch_bounds__(256) segment_sum_kernel(const T* __restrict__ in, const int64_t* __restrict__ ptr,
                                                          const int64_t* __restrict__ perm, T* __restrict__ out,
                                                          int64_t segments, int64_t width) {
  using A = typename Acc<T>::type;
  const int64_t total = segments * width;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t d = idx / width, c = idx % width;
    A acc = 0;
    for (int64_t e = __ldg(ptr + d); e < __ldg(ptr + d + 1); ++e) {
      const int64_t row = perm ? __ldg(perm + e) : e;
      acc += ld(in + row * width + c);
    }
    st(out + idx, acc);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) gather_rows_kernel(const T* __restrict__ in, const int64_t* __restrict__ index,
                                                          T* __restrict__ out, int64_t rows, int64_t width) {
  const int64_t total = rows * width;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x)
    out[idx] = in[__ldg(index + idx / width) * width + idx % width];
}

int check_table(const eqt_sh_table* t) {
  if (!t) return fail(EQT_ERR_BAD_ARGUMENT, "sh table is NULL");
  if (t->l_max < 0 || t->l_max > 64) return fail(EQT_ERR_UNSUPPORTED, "l_max %d outside [0, 64]", t->l_max);
  if (t->l_max > 0 && (!t->ptr || !t->m_out || !t->m_in || !t->axis || !t->coef))
    return fail(EQT_ERR_BAD_ARGUMENT, "sh table has NULL arrays");
  return EQT_OK;
}

template <typename T>
int sh_launch(bool backward, const void* xyz, const void* gout, void* out, int64_t n, const eqt_sh_table* t,
              int normalize, double out_scale, cudaStream_t s) {
  using A = typename Acc<T>::type;
  if (n == 0) return EQT_OK;
  switch (t->l_max) {   // straight-line kernels for the degrees generated at build time
    case 1: return sh_launch_unrolled<T, 1>(backward, xyz, gout, out, n, normalize, out_scale, s);
    case 2: return sh_launch_unrolled<T, 2>(backward, xyz, gout, out, n, normalize, out_scale, s);
    case 3: return sh_launch_unrolled<T, 3>(backward, xyz, gout, out, n, normalize, out_scale, s);
    case 4: return sh_launch_unrolled<T, 4>(backward, xyz, gout, out, n, normalize, out_scale, s);
    default: break;
  }
  ShTab tab{t->ptr, t->m_out, t->m_in, t->axis, t->coef, t->l_max};
  const int K = (t->l_max + 1) * (t->l_max + 1), W = 2 * t->l_max + 1;
  const size_t per_thread = sizeof(A) * (backward ? 8 * W : K);
  int threads = 256;
  while (threads > 32 && per_thread * threads > 64 * 1024) threads >>= 1;
  const size_t bytes = per_thread * threads;
  const unsigned grid = flat_grid(n, threads, 8);
  if (backward) {
    if (int rc = configure_smem(sh_backward_kernel<T>, bytes)) return rc;
    sh_backward_kernel<T><<<grid, threads, bytes, s>>>(static_cast<const T*>(xyz), static_cast<const T*>(gout),
                                                        static_cast<T*>(out), n, tab, normalize, (A)out_scale);
    return check_launch("sh_backward_kernel");
  }
  if (int rc = configure_smem(sh_forward_kernel<T>, bytes)) return rc;
  sh_forward_kernel<T><<<grid, threads, bytes, s>>>(static_cast<const T*>(xyz), static_cast<T*>(out), n, tab,
                                                     normalize, (A)out_scale);
  return check_launch("sh_forward_kernel");
}

}  // namespace
}  // namespace eqt

extern "C" int eqt_sh_forward(int32_t dtype, const void* xyz, void* out, int64_t n, const eqt_sh_table* table,
                              int32_t normalize, double out_scale, void* stream) {
  using namespace eqt;
  if (int rc = check_table(table)) return rc;
  if (n < 0 || (n > 0 && (!xyz || !out))) return fail(EQT_ERR_BAD_ARGUMENT, "bad xyz/out/n");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == EQT_F32) return sh_launch<float>(false, xyz, nullptr, out, n, table, normalize, out_scale, s);
  if (dtype == EQT_F64) return sh_launch<double>(false, xyz, nullptr, out, n, table, normalize, out_scale, s);
  return fail(EQT_ERR_UNSUPPORTED, "spherical harmonics support float32 and float64");
}

extern "C" int eqt_sh_backward(int32_t dtype, const void* xyz, const void* grad_out, void* grad_xyz, int64_t n,
                               const eqt_sh_table* table, int32_t normalize, double out_scale, void* stream) {
  using namespace eqt;
  if (int rc = check_table(table)) return rc;
  if (n < 0 || (n > 0 && (!xyz || !grad_out || !grad_xyz))) return fail(EQT_ERR_BAD_ARGUMENT, "bad pointers/n");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == EQT_F32) return sh_launch<float>(true, xyz, grad_out, grad_xyz, n, table, normalize, out_scale, s);
  if (dtype == EQT_F64) return sh_launch<double>(true, xyz, grad_out, grad_xyz, n, table, normalize, out_scale, s);
  return fail(EQT_ERR_UNSUPPORTED, "spherical harmonics support float32 and float64");
}

extern "C" int eqt_segment_sum(int32_t dtype, const void* in, const int64_t* ptr, const int64_t* perm, void* out,
                               int64_t num_segments, int64_t width, void* stream) {
  using namespace eqt;
  if (num_segments < 0 || width < 0) return fail(EQT_ERR_BAD_ARGUMENT, "negative size");
  if (num_segments == 0 || width == 0) return EQT_OK;
  if (!in || !ptr || !out) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = flat_grid(num_segments * width, 256);
  switch (dtype) {
    case EQT_F32: segment_sum_kernel<float><<<grid, 256, 0, s>>>((const float*)in, ptr, perm, (float*)out, num_segments, width); break;
    case EQT_F64: segment_sum_kernel<double><<<grid, 256, 0, s>>>((const double*)in, ptr, perm, (double*)out, num_segments, width); break;
    case EQT_BF16: segment_sum_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)in, ptr, perm, (__nv_bfloat16*)out, num_segments, width); break;
    default: return fail(EQT_ERR_BAD_ARGUMENT, "unknown dtype %d", dtype);
  }
  return check_launch("segment_sum_kernel");
}

extern "C" int eqt_gather_rows(int32_t dtype, const void* in, const int64_t* index, void* out, int64_t num_rows,
                               int64_t width, void* stream) {
  using namespace eqt;
  if (num_rows < 0 || width < 0) return fail(EQT_ERR_BAD_ARGUMENT, "negative size");
  if (num_rows == 0 || width == 0) return EQT_OK;
  if (!in || !index || !out) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = flat_grid(num_rows * width, 256);
  switch (dtype) {
    case EQT_F32: gather_rows_kernel<float><<<grid, 256, 0, s>>>((const float*)in, index, (float*)out, num_rows, width); break;
    case EQT_F64: gather_rows_kernel<double><<<grid, 256, 0, s>>>((const double*)in, index, (double*)out, num_rows, width); break;
    case EQT_BF16: gather_rows_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)in, index, (__nv_bfloat16*)out, num_rows, width); break;
    default: return fail(EQT_ERR_BAD_ARGUMENT, "unknown dtype %d", dtype);
  }
  return check_launch("gather_rows_kernel");
}
