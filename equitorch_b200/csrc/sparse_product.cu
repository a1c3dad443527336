// Generic batched sparse-dense products (table driven).
//
// One kernel family per product shape.  All of them read the sorted table
// (scale, index1, index2, seg, gather_index, index_out) straight from global memory: the
// loads are warp-uniform, so they are broadcast from L1.  The hot configurations of the
// tensor-product layers do not go through these kernels but through the fused ones in
// so3_fused.cu; these cover every flag combination of the operator API.
#include <algorithm>
#include <cstdarg>
#include <type_traits>

#include "common.cuh"

namespace eqt {

thread_local char t_error[512] = "";
std::atomic<int64_t> g_launches{0};
char* error_buffer() { return t_error; }
int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
  return code;
}
int sm_count() {
  constexpr int kMaxDevices = 64;
  static std::atomic<int> cached[kMaxDevices];   // zero-initialised; a race only repeats the query
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev >= 0 && dev < kMaxDevices) {
    const int n = cached[dev].load(std::memory_order_relaxed);
    if (n > 0) return n;
  }
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  if (dev >= 0 && dev < kMaxDevices) cached[dev].store(n, std::memory_order_relaxed);
  return n;
}

namespace {

struct P {  // kernel-side copy of eqt_product_args with strides resolved
  const void* in1;
  const void* in2;
  void* out;
  const void* scale;
  const int64_t* i1;
  const int64_t* i2;
  const int64_t* seg;
  const int64_t* gather;
  const int64_t* iout;
  int64_t n, rows1, rows2, num_out, out_size, c1, c2;
  int64_t bs1, bs2;  // batch strides in elements (0 when shared)
};

struct Entry {
  int64_t r1, r2, tt;
};

__device__ __forceinline__ void seg_range(const P& p, int64_t o, int64_t& t0, int64_t& t1) {
  if (p.seg) {
    t0 = __ldg(p.seg + o);
    t1 = __ldg(p.seg + o + 1);
  } else {
    t0 = o;
    t1 = o + 1;
  }
}
__device__ __forceinline__ Entry entry(const P& p, int64_t t) {
  Entry e;
  e.tt = p.gather ? __ldg(p.gather + t) : t;
  e.r1 = p.i1 ? __ldg(p.i1 + e.tt) : e.tt;
  e.r2 = p.i2 ? __ldg(p.i2 + e.tt) : e.tt;
  return e;
}
template <typename T>
__device__ __forceinline__ typename Acc<T>::type scale_of(const P& p, int64_t tt) {
  using A = typename Acc<T>::type;
  return p.scale ? __ldg(static_cast<const A*>(p.scale) + tt) : A(1);
}
__device__ __forceinline__ int64_t out_row(const P& p, int64_t o) { return p.iout ? __ldg(p.iout + o) : o; }

// ------------------------------------------------------------------------------------------
// channel-wise family: MUL, VECSCA, SCALE
// ------------------------------------------------------------------------------------------
template <typename T, int OP>
__global__ void __launch_bounds__(256) ew_kernel(P p) {
  using A = typename Acc<T>::type;
  const T* x = static_cast<const T*>(p.in1);
  const T* y = static_cast<const T*>(p.in2);
  T* out = static_cast<T*>(p.out);
  const int64_t C = p.c1;
  const int64_t total = p.n * p.num_out * C;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t c = idx % C;
    const int64_t o = (idx / C) % p.num_out;
    const int64_t n = idx / (C * p.num_out);
    int64_t t0, t1;
    seg_range(p, o, t0, t1);
    A acc = 0;
    for (int64_t t = t0; t < t1; ++t) {
      const Entry e = entry(p, t);
      A v = ld(x + n * p.bs1 + e.r1 * C + c);
      if (OP == EQT_OP_MUL) v *= ld(y + n * p.bs2 + e.r2 * C + c);
      if (OP == EQT_OP_VECSCA) v *= ld(y + n * p.bs2 + e.r2);
      acc += v * scale_of<T>(p, e.tt);
    }
    st(out + (n * p.out_size + out_row(p, o)) * C + c, acc);
  }
}

// float, C % 4 == 0, 16-byte aligned operands: four channels per thread, 128-bit accesses.
// I: index type of the flattened (sample, output row, channel group) loop; 32-bit when the count fits (64-bit
// divisions cost more than the loads of an element).
template <int OP, typename I>
__global__ void __launch_bounds__(256) ew_kernel_f4(P p) {
  const float* x = static_cast<const float*>(p.in1);
  const float* y = static_cast<const float*>(p.in2);
  float* out = static_cast<float*>(p.out);
  const int64_t C = p.c1;
  const I C4 = (I)(C / 4), num_out = (I)p.num_out;
  const I total = (I)(p.n * p.num_out * (C / 4));
  for (I idx = (I)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (I)gridDim.x * blockDim.x) {
    const int64_t c = (int64_t)(idx % C4) * 4;
    const int64_t o = (int64_t)((idx / C4) % num_out);
    const int64_t n = (int64_t)(idx / (C4 * num_out));
    int64_t t0, t1;
    seg_range(p, o, t0, t1);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int64_t t = t0; t < t1; ++t) {
      const Entry e = entry(p, t);
      float4 v = __ldg(reinterpret_cast<const float4*>(x + n * p.bs1 + e.r1 * C + c));
      float s = p.scale ? __ldg(static_cast<const float*>(p.scale) + e.tt) : 1.f;
      if (OP == EQT_OP_MUL) {
        const float4 w = __ldg(reinterpret_cast<const float4*>(y + n * p.bs2 + e.r2 * C + c));
        v.x *= w.x; v.y *= w.y; v.z *= w.z; v.w *= w.w;
      }
      if (OP == EQT_OP_VECSCA) s *= __ldg(y + n * p.bs2 + e.r2);
      acc.x += v.x * s; acc.y += v.y * s; acc.z += v.z * s; acc.w += v.w * s;
    }
    *reinterpret_cast<float4*>(out + (n * p.out_size + out_row(p, o)) * C + c) = acc;
  }
}

// bfloat16 storage, C % 8 == 0, 16-byte aligned operands: eight channels per thread, 128-bit accesses, float sums,
// 32-bit index arithmetic (the launcher checks that the element count fits).
template <int OP>
__global__ void __launch_bounds__(256) ew_kernel_b8(P p) {
  const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(p.in1);
  const __nv_bfloat16* y = static_cast<const __nv_bfloat16*>(p.in2);
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
  const uint32_t C = (uint32_t)p.c1, C8 = C / 8, num_out = (uint32_t)p.num_out;
  const uint32_t total = (uint32_t)p.n * num_out * C8;
  for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
    const uint32_t c = (idx % C8) * 8;
    const uint32_t o = (idx / C8) % num_out;
    const int64_t n = idx / (C8 * num_out);
    int64_t t0, t1;
    seg_range(p, o, t0, t1);
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int64_t t = t0; t < t1; ++t) {
      const Entry e = entry(p, t);
      const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + n * p.bs1 + e.r1 * C + c));
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
      float s = p.scale ? __ldg(static_cast<const float*>(p.scale) + e.tt) : 1.f;
      float v[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(xp[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
      }
      if (OP == EQT_OP_MUL) {
        const uint4 yv = __ldg(reinterpret_cast<const uint4*>(y + n * p.bs2 + e.r2 * C + c));
        const __nv_bfloat162* yp = reinterpret_cast<const __nv_bfloat162*>(&yv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(yp[i]);
          v[2 * i] *= f.x;
          v[2 * i + 1] *= f.y;
        }
      }
      if (OP == EQT_OP_VECSCA) s *= __bfloat162float(__ldg(y + n * p.bs2 + e.r2));
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += v[i] * s;
    }
    uint4 ov;
    __nv_bfloat162* op2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int i = 0; i < 4; ++i) op2[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    *reinterpret_cast<uint4*>(out + (n * p.out_size + out_row(p, o)) * C + c) = ov;
  }
}

// Batch-summed form: out[o, c] = sum_n sum_t ...   block = 32 channels x 8 batch lanes,
// grid = (num_out * channel tiles, batch chunks); one atomicAdd per block and output element.
template <typename T, int OP>
__global__ void __launch_bounds__(256) ew_acc_kernel(P p, int64_t chunk) {
  using A = typename Acc<T>::type;
  __shared__ A red[8][33];
  const T* x = static_cast<const T*>(p.in1);
  const T* y = static_cast<const T*>(p.in2);
  A* out = static_cast<A*>(p.out);
  const int64_t C = p.c1;
  const int64_t ctiles = ceil_div(C, 32);
  const int64_t o = blockIdx.x / ctiles;
  const int64_t c = (blockIdx.x % ctiles) * 32 + threadIdx.x;
  const int64_t n0 = blockIdx.y * chunk;
  const int64_t n1 = min(n0 + chunk, p.n);
  int64_t t0, t1;
  seg_range(p, o, t0, t1);
  A acc = 0;
  // The entries of the output row are the same for every sample: they are staged in shared memory once (up to
  // ACC_STAGE of them), and four samples are in flight per thread - with one, a thread waited for the latency of
  // memory at every sample and the kernel ran at a seventh of the bandwidth.
  constexpr int ACC_STAGE = 64;
  __shared__ int32_t e_r1[ACC_STAGE], e_r2[ACC_STAGE];
  __shared__ A e_sc[ACC_STAGE];
  const bool staged = t1 - t0 <= ACC_STAGE;
  if (staged) {
    const int tid = threadIdx.y * 32 + threadIdx.x;
    if (tid < t1 - t0) {
      const Entry e = entry(p, t0 + tid);
      e_r1[tid] = (int32_t)e.r1;
      e_r2[tid] = (int32_t)e.r2;
      e_sc[tid] = scale_of<T>(p, e.tt);
    }
    __syncthreads();
  }
  if (c < C && staged) {
    const int ne = (int)(t1 - t0);
    for (int64_t n = n0 + threadIdx.y; n < n1; n += 32) {
      A part[4] = {0, 0, 0, 0};
      for (int t = 0; t < ne; ++t) {
        const int64_t o1 = (int64_t)e_r1[t] * C + c, o2 = OP == EQT_OP_MUL ? (int64_t)e_r2[t] * C + c : (int64_t)e_r2[t];
        const A sc = e_sc[t];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int64_t nn = n + 8 * u;
          if (nn < n1) {
            A v = ld(x + nn * p.bs1 + o1);
            if (OP == EQT_OP_MUL || OP == EQT_OP_VECSCA) v *= ld(y + nn * p.bs2 + o2);
            part[u] += v * sc;
          }
        }
      }
      acc += (part[0] + part[1]) + (part[2] + part[3]);
    }
  } else if (c < C) {
    for (int64_t n = n0 + threadIdx.y; n < n1; n += 8) {
      for (int64_t t = t0; t < t1; ++t) {
        const Entry e = entry(p, t);
        A v = ld(x + n * p.bs1 + e.r1 * C + c);
        if (OP == EQT_OP_MUL) v *= ld(y + n * p.bs2 + e.r2 * C + c);
        if (OP == EQT_OP_VECSCA) v *= ld(y + n * p.bs2 + e.r2);
        acc += v * scale_of<T>(p, e.tt);
      }
    }
  }
  red[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && c < C) {
    A s = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += red[k][threadIdx.x];
    atomicAdd(out + out_row(p, o) * C + c, s);
  }
}

// ------------------------------------------------------------------------------------------
// OUTER
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) outer_kernel(P p) {
  using A = typename Acc<T>::type;
  const T* x = static_cast<const T*>(p.in1);
  const T* y = static_cast<const T*>(p.in2);
  T* out = static_cast<T*>(p.out);
  const int64_t C1 = p.c1, C2 = p.c2, CC = C1 * C2;
  const int64_t total = p.n * p.num_out * CC;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t b = idx % C2;
    const int64_t a = (idx / C2) % C1;
    const int64_t o = (idx / CC) % p.num_out;
    const int64_t n = idx / (CC * p.num_out);
    int64_t t0, t1;
    seg_range(p, o, t0, t1);
    A acc = 0;
    for (int64_t t = t0; t < t1; ++t) {
      const Entry e = entry(p, t);
      acc += ld(x + n * p.bs1 + e.r1 * C1 + a) * ld(y + n * p.bs2 + e.r2 * C2 + b) * scale_of<T>(p, e.tt);
    }
    st(out + (n * p.out_size + out_row(p, o)) * CC + idx % CC, acc);
  }
}

// Batch-summed outer product = a GEMM whose reduction runs over (sample, table entry) pairs:
//   out[o, a, b] = sum_{n, t in seg[o]} s_t x[n, i1_t, a] y[n, i2_t, b].
// 64x64 output tile per block, 4x4 per thread, 8 pairs staged in shared memory per step.
// grid = (tiles_a * tiles_b, num_out, batch chunks); partial tiles are combined with atomicAdd.
template <typename T>
__global__ void __launch_bounds__(256) outer_acc_kernel(P p, int64_t chunk) {
  using A = typename Acc<T>::type;
  constexpr int TILE = 64, KK = 8;
  __shared__ A sa[KK][TILE];
  __shared__ A sb[KK][TILE];
  const T* x = static_cast<const T*>(p.in1);
  const T* y = static_cast<const T*>(p.in2);
  A* out = static_cast<A*>(p.out);
  const int64_t C1 = p.c1, C2 = p.c2;
  const int64_t tiles_b = ceil_div(C2, TILE);
  const int64_t a0 = (blockIdx.x / tiles_b) * TILE, b0 = (blockIdx.x % tiles_b) * TILE;
  const int64_t o = blockIdx.y;
  const int64_t n0 = blockIdx.z * chunk, n1 = min(n0 + chunk, p.n);
  int64_t t0, t1;
  seg_range(p, o, t0, t1);
  const int64_t len = t1 - t0;
  const int64_t pairs = (n1 - n0) * len;
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  A acc[4][4] = {};
  for (int64_t k0 = 0; k0 < pairs; k0 += KK) {
    // 2 * KK * TILE = 1024 loads for 256 threads
    for (int q = tid; q < 2 * KK * TILE; q += 256) {
      const int which = q / (KK * TILE), r = (q / TILE) % KK, col = q % TILE;
      const int64_t k = k0 + r;
      A v = 0;
      if (k < pairs) {
        const int64_t n = n0 + k / len;
        const Entry e = entry(p, t0 + k % len);
        if (which == 0) {
          if (a0 + col < C1) v = ld(x + n * p.bs1 + e.r1 * C1 + a0 + col) * scale_of<T>(p, e.tt);
        } else {
          if (b0 + col < C2) v = ld(y + n * p.bs2 + e.r2 * C2 + b0 + col);
        }
      }
      (which == 0 ? sa : sb)[r][col] = v;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < KK; ++r) {
      A av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = sa[r][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = sb[r][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
    }
    __syncthreads();
  }
  const int64_t orow = out_row(p, o);
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t a = a0 + ty * 4 + i, b = b0 + tx * 4 + j;
      if (a < C1 && b < C2 && pairs > 0) atomicAdd(out + (orow * C1 + a) * C2 + b, acc[i][j]);
    }
}

// ------------------------------------------------------------------------------------------
// INNER: one warp per (sample, output row)
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) inner_kernel(P p, int accumulated) {
  using A = typename Acc<T>::type;
  const T* x = static_cast<const T*>(p.in1);
  const T* y = static_cast<const T*>(p.in2);
  const int64_t C = p.c1;
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int64_t total = p.n * p.num_out;
  for (int64_t w = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5); w < total; w += warps) {
    const int64_t o = w % p.num_out, n = w / p.num_out;
    int64_t t0, t1;
    seg_range(p, o, t0, t1);
    A acc = 0;
    for (int64_t t = t0; t < t1; ++t) {
      const Entry e = entry(p, t);
      const T* xr = x + n * p.bs1 + e.r1 * C;
      const T* yr = y + n * p.bs2 + e.r2 * C;
      A dot = 0;
      for (int64_t c = lane; c < C; c += 32) dot += ld(xr + c) * ld(yr + c);
      acc += dot * scale_of<T>(p, e.tt);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) {
      const int64_t orow = out_row(p, o);
      if (accumulated)
        atomicAdd(static_cast<A*>(p.out) + orow, acc);
      else
        st(static_cast<T*>(p.out) + n * p.out_size + orow, acc);
    }
  }
}

// ------------------------------------------------------------------------------------------
// VECMAT
// ------------------------------------------------------------------------------------------
// Weights shared by the batch, output per sample: a grouped GEMM.  Block = 64 samples x 64
// output channels of one output row; the reduction runs over (table entry, input channel).
template <typename T>
__global__ void __launch_bounds__(256) vecmat_shared_w_kernel(P p) {
  using A = typename Acc<T>::type;
  constexpr int BN = 64, BCO = 64, KC = 16, PAD = 4;
  __shared__ A sx[KC][BN + PAD];
  __shared__ A sw[KC][BCO];
  const T* x = static_cast<const T*>(p.in1);
  const T* w = static_cast<const T*>(p.in2);
  T* out = static_cast<T*>(p.out);
  const int64_t Cin = p.c1, Cout = p.c2;
  const int64_t cotiles = ceil_div(Cout, BCO);
  const int64_t n0 = (blockIdx.x / cotiles) * BN, co0 = (blockIdx.x % cotiles) * BCO;
  const int64_t o = blockIdx.y;
  int64_t t0, t1;
  seg_range(p, o, t0, t1);
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  A acc[4][4] = {};
  for (int64_t t = t0; t < t1; ++t) {
    const Entry e = entry(p, t);
    const A s = scale_of<T>(p, e.tt);
    for (int64_t ci0 = 0; ci0 < Cin; ci0 += KC) {
      for (int q = tid; q < KC * BN; q += 256) {  // x tile, transposed on the way in
        const int nn = q / KC, k = q % KC;
        A v = 0;
        if (n0 + nn < p.n && ci0 + k < Cin) v = ld(x + (n0 + nn) * p.bs1 + e.r1 * Cin + ci0 + k) * s;
        sx[k][nn] = v;
      }
      for (int q = tid; q < KC * BCO; q += 256) {
        const int k = q / BCO, j = q % BCO;
        A v = 0;
        if (ci0 + k < Cin && co0 + j < Cout) v = ld(w + (e.r2 * Cin + ci0 + k) * Cout + co0 + j);
        sw[k][j] = v;
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < KC; ++k) {
        A av[4], bv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) av[i] = sx[k][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[j] = sw[k][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
      }
      __syncthreads();
    }
  }
  const int64_t orow = out_row(p, o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t n = n0 + ty * 4 + i;
    if (n >= p.n) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t co = co0 + tx * 4 + j;
      if (co < Cout) st(out + (n * p.out_size + orow) * Cout + co, acc[i][j]);
    }
  }
}

// Any other sharing pattern (per-sample matrices, shared vector, batch-summed output): one
// thread per output element; the matrix is streamed once, so this form is bandwidth bound.
template <typename T>
__global__ void __launch_bounds__(256) vecmat_direct_kernel(P p, int accumulated) {
  using A = typename Acc<T>::type;
  const T* x = static_cast<const T*>(p.in1);
  const T* w = static_cast<const T*>(p.in2);
  const int64_t Cin = p.c1, Cout = p.c2;
  const int64_t total = p.n * p.num_out * Cout;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t co = idx % Cout;
    const int64_t o = (idx / Cout) % p.num_out;
    const int64_t n = idx / (Cout * p.num_out);
    int64_t t0, t1;
    seg_range(p, o, t0, t1);
    A acc = 0;
    for (int64_t t = t0; t < t1; ++t) {
      const Entry e = entry(p, t);
      const T* xr = x + n * p.bs1 + e.r1 * Cin;
      const T* wr = w + n * p.bs2 + e.r2 * Cin * Cout + co;
      A dot = 0;
      for (int64_t ci = 0; ci < Cin; ++ci) dot += ld(xr + ci) * ld(wr + ci * Cout);
      acc += dot * scale_of<T>(p, e.tt);
    }
    const int64_t orow = out_row(p, o);
    if (accumulated)
      atomicAdd(static_cast<A*>(p.out) + orow * Cout + co, acc);
    else
      st(static_cast<T*>(p.out) + (n * p.out_size + orow) * Cout + co, acc);
  }
}

// ------------------------------------------------------------------------------------------
// dispatch
// ------------------------------------------------------------------------------------------
inline bool aligned16(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; }

template <typename T>
int launch(const eqt_product_args& a, P p, cudaStream_t s) {
  const int op = a.op;
  if (p.n == 0 || p.num_out == 0) return EQT_OK;
  if (op == EQT_OP_MUL || op == EQT_OP_VECSCA || op == EQT_OP_SCALE) {
    if (p.c1 == 0) return EQT_OK;
    if (a.accumulated) {
      const int64_t blocks_x = p.num_out * ceil_div(p.c1, 32);
      int64_t chunks = ceil_div((int64_t)sm_count() * 8, blocks_x);
      chunks = std::max<int64_t>(1, std::min<int64_t>(chunks, ceil_div(p.n, 64)));
      chunks = std::min<int64_t>(chunks, 65535);
      const int64_t chunk = ceil_div(p.n, chunks);
      dim3 grid((unsigned)blocks_x, (unsigned)ceil_div(p.n, chunk)), block(32, 8);
      if (op == EQT_OP_MUL) ew_acc_kernel<T, EQT_OP_MUL><<<grid, block, 0, s>>>(p, chunk);
      if (op == EQT_OP_VECSCA) ew_acc_kernel<T, EQT_OP_VECSCA><<<grid, block, 0, s>>>(p, chunk);
      if (op == EQT_OP_SCALE) ew_acc_kernel<T, EQT_OP_SCALE><<<grid, block, 0, s>>>(p, chunk);
      return check_launch("ew_acc_kernel");
    }
    if (std::is_same<T, float>::value && p.c1 % 4 == 0 && aligned16(p.in1) && aligned16(p.out) &&
        (op != EQT_OP_MUL || aligned16(p.in2))) {
      const int64_t work = p.n * p.num_out * (p.c1 / 4);
      const unsigned grid = flat_grid(work, 256);
      if (work + (int64_t)grid * 256 < (int64_t(1) << 32)) {      // the strided index cannot wrap
        if (op == EQT_OP_MUL) ew_kernel_f4<EQT_OP_MUL, uint32_t><<<grid, 256, 0, s>>>(p);
        if (op == EQT_OP_VECSCA) ew_kernel_f4<EQT_OP_VECSCA, uint32_t><<<grid, 256, 0, s>>>(p);
        if (op == EQT_OP_SCALE) ew_kernel_f4<EQT_OP_SCALE, uint32_t><<<grid, 256, 0, s>>>(p);
      } else {
        if (op == EQT_OP_MUL) ew_kernel_f4<EQT_OP_MUL, int64_t><<<grid, 256, 0, s>>>(p);
        if (op == EQT_OP_VECSCA) ew_kernel_f4<EQT_OP_VECSCA, int64_t><<<grid, 256, 0, s>>>(p);
        if (op == EQT_OP_SCALE) ew_kernel_f4<EQT_OP_SCALE, int64_t><<<grid, 256, 0, s>>>(p);
      }
      return check_launch("ew_kernel_f4");
    }
    if (std::is_same<T, __nv_bfloat16>::value && p.c1 % 8 == 0 && aligned16(p.in1) && aligned16(p.out) &&
        (op != EQT_OP_MUL || aligned16(p.in2)) && p.n * p.num_out * (p.c1 / 8) < (int64_t(1) << 31)) {
      const unsigned grid = flat_grid(p.n * p.num_out * (p.c1 / 8), 256);
      if (op == EQT_OP_MUL) ew_kernel_b8<EQT_OP_MUL><<<grid, 256, 0, s>>>(p);
      if (op == EQT_OP_VECSCA) ew_kernel_b8<EQT_OP_VECSCA><<<grid, 256, 0, s>>>(p);
      if (op == EQT_OP_SCALE) ew_kernel_b8<EQT_OP_SCALE><<<grid, 256, 0, s>>>(p);
      return check_launch("ew_kernel_b8");
    }
    const unsigned grid = flat_grid(p.n * p.num_out * p.c1, 256);
    if (op == EQT_OP_MUL) ew_kernel<T, EQT_OP_MUL><<<grid, 256, 0, s>>>(p);
    if (op == EQT_OP_VECSCA) ew_kernel<T, EQT_OP_VECSCA><<<grid, 256, 0, s>>>(p);
    if (op == EQT_OP_SCALE) ew_kernel<T, EQT_OP_SCALE><<<grid, 256, 0, s>>>(p);
    return check_launch("ew_kernel");
  }
  if (op == EQT_OP_OUTER) {
    if (p.c1 == 0 || p.c2 == 0) return EQT_OK;
    if (a.accumulated) {
      const int64_t tiles = ceil_div(p.c1, 64) * ceil_div(p.c2, 64);
      if (p.num_out > 65535) return fail(EQT_ERR_UNSUPPORTED, "accumulated outer: more than 65535 output rows");
      int64_t chunks = ceil_div((int64_t)sm_count() * 4, tiles * p.num_out);
      chunks = std::max<int64_t>(1, std::min<int64_t>(chunks, ceil_div(p.n, 32)));
      chunks = std::min<int64_t>(chunks, 65535);
      const int64_t chunk = ceil_div(p.n, chunks);
      dim3 grid((unsigned)tiles, (unsigned)p.num_out, (unsigned)ceil_div(p.n, chunk));
      outer_acc_kernel<T><<<grid, 256, 0, s>>>(p, chunk);
      return check_launch("outer_acc_kernel");
    }
    outer_kernel<T><<<flat_grid(p.n * p.num_out * p.c1 * p.c2, 256), 256, 0, s>>>(p);
    return check_launch("outer_kernel");
  }
  if (op == EQT_OP_INNER) {
    inner_kernel<T><<<flat_grid(p.n * p.num_out, 8), 256, 0, s>>>(p, a.accumulated);
    return check_launch("inner_kernel");
  }
  if (op == EQT_OP_VECMAT) {
    if (p.c2 == 0) return EQT_OK;
    if (a.shared2 && !a.shared1 && !a.accumulated && p.num_out <= 65535) {
      dim3 grid((unsigned)(ceil_div(p.n, 64) * ceil_div(p.c2, 64)), (unsigned)p.num_out);
      vecmat_shared_w_kernel<T><<<grid, 256, 0, s>>>(p);
      return check_launch("vecmat_shared_w_kernel");
    }
    vecmat_direct_kernel<T><<<flat_grid(p.n * p.num_out * p.c2, 256), 256, 0, s>>>(p, a.accumulated);
    return check_launch("vecmat_direct_kernel");
  }
  return fail(EQT_ERR_BAD_ARGUMENT, "unknown op %d", op);
}

}  // namespace
}  // namespace eqt

extern "C" int eqt_sparse_product(const eqt_product_args* a, void* stream) {
  using namespace eqt;
  if (!a) return fail(EQT_ERR_BAD_ARGUMENT, "args is NULL");
  if (a->n < 0 || a->num_out < 0 || a->out_size < 0 || a->c1 < 0 || a->c2 < 0 || a->rows1 < 0 || a->rows2 < 0)
    return fail(EQT_ERR_BAD_ARGUMENT, "negative size");
  const bool empty = a->n == 0 || a->num_out == 0;
  if (!empty && (!a->in1 || !a->out || (a->op != EQT_OP_SCALE && !a->in2)))
    return fail(EQT_ERR_BAD_ARGUMENT, "NULL operand");
  if (a->op == EQT_OP_SCALE && a->accumulated == 0 && a->shared1)
    return fail(EQT_ERR_BAD_ARGUMENT, "scale-segment needs a batched input");
  P p;
  p.in1 = a->in1; p.in2 = a->in2; p.out = a->out; p.scale = a->scale;
  p.i1 = a->index1; p.i2 = a->index2; p.seg = a->seg; p.gather = a->gather_index; p.iout = a->index_out;
  p.n = a->n; p.rows1 = a->rows1; p.rows2 = a->rows2; p.num_out = a->num_out; p.out_size = a->out_size;
  p.c1 = a->c1; p.c2 = a->c2;
  p.bs1 = a->shared1 ? 0 : a->rows1 * a->c1;
  switch (a->op) {
    case EQT_OP_MUL: case EQT_OP_INNER: p.bs2 = a->rows2 * a->c1; break;
    case EQT_OP_VECSCA: p.bs2 = a->rows2; break;
    case EQT_OP_OUTER: p.bs2 = a->rows2 * a->c2; break;
    case EQT_OP_VECMAT: p.bs2 = a->rows2 * a->c1 * a->c2; break;
    case EQT_OP_SCALE: p.bs2 = 0; break;
    default: return fail(EQT_ERR_BAD_ARGUMENT, "unknown op %d", a->op);
  }
  if (a->shared2) p.bs2 = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (a->dtype) {
    case EQT_F32: return launch<float>(*a, p, s);
    case EQT_F64: return launch<double>(*a, p, s);
    case EQT_BF16: return launch<__nv_bfloat16>(*a, p, s);
    default: return fail(EQT_ERR_BAD_ARGUMENT, "unknown dtype %d", a->dtype);
  }
}

extern "C" const char* eqt_last_error(void) { return eqt::error_buffer(); }
extern "C" int eqt_version(void) { return 100; }
extern "C" int64_t eqt_launch_count(void) { return eqt::g_launches.load(); }
