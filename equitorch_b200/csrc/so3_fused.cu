// Fused Clebsch-Gordan kernels of the graph tensor-product layer (float32).
//
//   tp_cg_segment_sum:  S[d, r, c] = sum_{e in seg[d]} sum_{t in row r} scale[t] * y[e, my[t]] * feat[fidx[e], mf[t], c]
//   tp_cg_inner:        gy[e, k]   = sum_{t: my[t] = k} scale[t] * sum_c feat[fidx[e], mf[t], c] * G[node(e), row[t], c]
//
// i.e. gather of node rows by edge, CG contraction with the edge's spherical harmonics and the
// sum over the edges of a destination node in one pass - the per-edge intermediate (99 x 64
// floats for l_max = 3) never reaches HBM - and the adjoint needed for the gradient with
// respect to the harmonics.
//
// Two implementations of each:
//  * "spec": for index structures unrolled at build time (generated/tp_specs.inc).  One CTA of
//    four warps walks a contiguous range of destination nodes.  Feature rows of the next four
//    edges are fetched with bulk asynchronous copies (cp.async.bulk + mbarrier, double
//    buffered) while the current four are consumed.  Each warp owns a contiguous block of
//    intermediate rows; a lane holds CPL channels of all D_feat gathered components and of its
//    rows' accumulators in registers, the per-edge coefficients scale[t]*y[my[t]] are built
//    by the warp in shared memory and read back as broadcast 128-bit loads.  No atomics: the
//    edges of a node are consecutive, the accumulators are flushed once per node.
//  * "generic": table-driven, one thread per output element; any structure, any channel count.
#include <algorithm>

#include "common.cuh"

namespace eqt {
namespace specs {
#define EQT_FMA_ROW(ACC, A, X)                     \
  do {                                             \
    _Pragma("unroll") for (int k_ = 0; k_ < CPL; ++k_)(ACC)[k_] = fmaf((A), (X)[k_], (ACC)[k_]); \
  } while (0)
template <int CPL>
__device__ __forceinline__ float dot_row(const float (&a)[CPL], const float (&b)[CPL]) {
  float s = a[0] * b[0];
#pragma unroll
  for (int k = 1; k < CPL; ++k) s = fmaf(a[k], b[k], s);
  return s;
}
#define EQT_DOT_ROW(X, G) dot_row<CPL>((X), (G))
#include "generated/tp_specs.inc"
#undef EQT_FMA_ROW
#undef EQT_DOT_ROW
}  // namespace specs

namespace {

constexpr int STAGES = 4;   // edges per batch
constexpr int NW = 4;       // warps per CTA
constexpr int WAIT_SPINS = 1 << 22;

struct FusedArgs {
  const float* feat;        // (rows, DF, C)
  const int64_t* fidx;      // (E) feature row of each edge, or NULL (= e)
  const float* y;           // (Ey, DY)
  const int64_t* yidx;      // (E) row of y (and of grad_y) of each edge, or NULL (= e)
  const int64_t* ptr;       // (N + 1) CSR of edges per output node, or NULL (one edge per output)
  const int64_t* enode;     // (E) node of each edge (generic inner kernel only)
  const float* scale;       // (T)
  const float* scale_k;     // (T) in the unrolled kernels' entry order, or NULL
  const int64_t* my_k;      // (T) likewise
  const int64_t* mf;        // (T)
  const int64_t* my;        // (T)
  const int64_t* rowptr;    // (R + 1)
  const float* g;           // (N, R, C)  inner only
  float* out;               // segsum: (N, R, C); inner: (Ey, DY)
  int64_t n_out, n_edges;
  int T, R, DF, DY, C;
  int nodes_per_cta;
  int* status;
};

// ---- PTX wrappers --------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after WAIT_SPINS polls so that a lost copy cannot hang the GPU.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (int i = 0; i < WAIT_SPINS; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 32) __nanosleep(64);
  }
  return false;
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}
__device__ __forceinline__ void cta_sync() { asm volatile("bar.sync 0;" ::: "memory"); }

template <class S>
__device__ __forceinline__ void warp_ranges(int w, int& tb, int& te, int& rb, int& re) {
  tb = S::WT[0]; te = S::WT[1]; rb = S::WR[0]; re = S::WR[1];
  if (w == 1) { tb = S::WT[1]; te = S::WT[2]; rb = S::WR[1]; re = S::WR[2]; }
  if (w == 2) { tb = S::WT[2]; te = S::WT[3]; rb = S::WR[2]; re = S::WR[3]; }
  if (w == 3) { tb = S::WT[3]; te = S::WT[4]; rb = S::WR[3]; re = S::WR[4]; }
}

template <class S, int CPL>
constexpr size_t spec_smem_bytes() {
  return sizeof(float) * (2 * STAGES * S::DF * 32 * CPL   // feature rows, two sets
                          + 2 * NW * S::MAXT              // per-warp coefficients and scales
                          + NW * STAGES * S::DY           // per-warp copy of the batch's harmonics
                          + 2 * STAGES * NW * S::DY)      // inner: per-warp partial grad_y, two sets
         + S::T                                           // my[] as bytes
         + 64;
}

// Shared prologue: carve shared memory, stage the per-warp scale block and my[], init barriers.
template <class S, int CPL>
struct Smem {
  float* xs;
  float* wbuf;    // [NW][MAXT] coefficients of the current edge
  float* wsc;     // [NW][MAXT] scales of the warp's entries
  float* wy;      // [NW][STAGES][DY]
  float* red;     // [2][STAGES][NW][DY]
  uint8_t* smy;   // [T]
  __device__ explicit Smem(unsigned char* base) {
    xs = reinterpret_cast<float*>(base);
    wbuf = xs + 2 * STAGES * S::DF * 32 * CPL;
    wsc = wbuf + NW * S::MAXT;
    wy = wsc + NW * S::MAXT;
    red = wy + NW * STAGES * S::DY;
    smy = reinterpret_cast<uint8_t*>(red + 2 * STAGES * NW * S::DY);
  }
};

// ---- spec kernel: gather + CG + segment sum -----------------------------------------------------
template <class S, int CPL>
__global__ void __launch_bounds__(NW * 32, 4) tp_segsum_spec_kernel(FusedArgs a) {
  constexpr int C = 32 * CPL, ROWF = S::DF * C;
  constexpr uint32_t ROWB = ROWF * sizeof(float);
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ uint64_t bars[2];
  Smem<S, CPL> sm(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int tb, te, rb, re;
  warp_ranges<S>(warp, tb, te, rb, re);
  float* wcoef = sm.wbuf + warp * S::MAXT;
  float* wscale = sm.wsc + warp * S::MAXT;
  float* wys = sm.wy + warp * STAGES * S::DY;

  for (int t = tid; t < S::T; t += NW * 32) sm.smy[t] = static_cast<uint8_t>(__ldg(a.my_k + t));
  for (int t = tb + lane; t < te; t += 32) wscale[t - tb] = __ldg(a.scale_k + t);
  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  cta_sync();

  const int64_t d0 = (int64_t)blockIdx.x * a.nodes_per_cta;
  const int64_t d1 = min(d0 + a.nodes_per_cta, a.n_out);
  const int64_t e0 = a.ptr ? __ldg(a.ptr + d0) : d0;
  const int64_t e1 = a.ptr ? __ldg(a.ptr + d1) : d1;
  const int64_t nb = ceil_div(e1 - e0, STAGES);

  auto issue = [&](int64_t b) {
    if (tid == 0) {
      const int set = b & 1;
      const int64_t eb = e0 + b * STAGES;
      const int cnt = (int)min((int64_t)STAGES, e1 - eb);
      mbar_expect_tx(&bars[set], cnt * ROWB);
      for (int s = 0; s < cnt; ++s) {
        const int64_t row = a.fidx ? __ldg(a.fidx + eb + s) : eb + s;
        bulk_load(sm.xs + (set * STAGES + s) * ROWF, a.feat + row * ROWF, ROWB, &bars[set]);
      }
    }
  };

  float acc[S::MAXR][CPL];
#pragma unroll
  for (int r = 0; r < S::MAXR; ++r)
#pragma unroll
    for (int k = 0; k < CPL; ++k) acc[r][k] = 0.f;

  int64_t d_cur = d0;
  int64_t boundary = a.ptr ? __ldg(a.ptr + d_cur + 1) : d_cur + 1;
  auto flush = [&]() {
    float* o = a.out + (d_cur * S::R + rb) * C + lane * CPL;
#pragma unroll
    for (int r = 0; r < S::MAXR; ++r) {
      if (r < re - rb) {
        if (CPL == 2) *reinterpret_cast<float2*>(o + r * C) = make_float2(acc[r][0], acc[r][CPL - 1]);
        else o[r * C] = acc[r][0];
      }
#pragma unroll
      for (int k = 0; k < CPL; ++k) acc[r][k] = 0.f;
    }
    ++d_cur;
    if (d_cur < d1) boundary = a.ptr ? __ldg(a.ptr + d_cur + 1) : d_cur + 1;
  };

  bool failed = false;
  if (nb > 0) issue(0);
  for (int64_t b = 0; b < nb; ++b) {
    if (b + 1 < nb) issue(b + 1);
    const int set = b & 1;
    const int64_t eb = e0 + b * STAGES;
    const int cnt = (int)min((int64_t)STAGES, e1 - eb);
    // the warp's own copy of the batch's harmonics (requested before waiting for the feature rows)
    for (int q = lane; q < cnt * S::DY; q += 32) {
      const int64_t e = eb + q / S::DY;
      wys[q] = __ldg(a.y + (a.yidx ? __ldg(a.yidx + e) : e) * S::DY + q % S::DY);
    }
    if (!mbar_wait(&bars[set], (b >> 1) & 1)) { failed = true; break; }
    __syncwarp();
    for (int s = 0; s < cnt; ++s) {
      const int64_t e = eb + s;
      while (e >= boundary) flush();
      const float* ye = wys + s * S::DY;
      for (int t = tb + lane; t < te; t += 32) wcoef[t - tb] = wscale[t - tb] * ye[sm.smy[t]];
      __syncwarp();
      float x[S::DF][CPL];
      const float* xr = sm.xs + (set * STAGES + s) * ROWF + lane * CPL;
#pragma unroll
      for (int m = 0; m < S::DF; ++m) {
        if (CPL == 2) {
          const float2 v = *reinterpret_cast<const float2*>(xr + m * C);
          x[m][0] = v.x; x[m][CPL - 1] = v.y;
        } else {
          x[m][0] = xr[m * C];
        }
      }
      const float4* cf = reinterpret_cast<const float4*>(wcoef);
      if (warp == 0) S::template segsum_w0<CPL>(acc, x, cf);
      else if (warp == 1) S::template segsum_w1<CPL>(acc, x, cf);
      else if (warp == 2) S::template segsum_w2<CPL>(acc, x, cf);
      else S::template segsum_w3<CPL>(acc, x, cf);
      __syncwarp();
    }
    cta_sync();   // everybody is done with this set before it is refilled
  }
  if (failed) {
    if (tid == 0) atomicExch(a.status, 1);
    // give copies that may still be in flight a bounded chance to land before the CTA retires
    mbar_wait(&bars[0], 0);
    mbar_wait(&bars[1], 0);
    return;
  }
  while (d_cur < d1) flush();
}

// Sum each of the N per-lane values over the 32 lanes and store the N totals.  For N = 16 the
// butterfly halves the number of live values at every step (8 + 4 + 2 + 1 + 1 shuffles instead of 80).
template <int N>
__device__ __forceinline__ void warp_reduce_to_smem(float (&v)[N], float* dst, int lane) {
  if constexpr (N == 16) {
    float a8[8], a4[4], a2[2];
    const bool h16 = lane & 16, h8 = lane & 8, h4 = lane & 4, h2 = lane & 2;
#pragma unroll
    for (int i = 0; i < 8; ++i) a8[i] = (h16 ? v[i + 8] : v[i]) + __shfl_xor_sync(0xffffffffu, h16 ? v[i] : v[i + 8], 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) a4[i] = (h8 ? a8[i + 4] : a8[i]) + __shfl_xor_sync(0xffffffffu, h8 ? a8[i] : a8[i + 4], 8);
#pragma unroll
    for (int i = 0; i < 2; ++i) a2[i] = (h4 ? a4[i + 2] : a4[i]) + __shfl_xor_sync(0xffffffffu, h4 ? a4[i] : a4[i + 2], 4);
    float r = (h2 ? a2[1] : a2[0]) + __shfl_xor_sync(0xffffffffu, h2 ? a2[0] : a2[1], 2);
    r += __shfl_xor_sync(0xffffffffu, r, 1);
    // lane bits (16, 8, 4, 2) select which of the 16 values this lane ended up with
    if ((lane & 1) == 0) dst[(h16 ? 8 : 0) + (h8 ? 4 : 0) + (h4 ? 2 : 0) + (h2 ? 1 : 0)] = r;
  } else {
#pragma unroll
    for (int k = 0; k < N; ++k) {
      float t = v[k];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      if (lane == 0) dst[k] = t;
    }
  }
}

// ---- spec kernel: adjoint w.r.t. the channel-less operand ----------------------------------------
template <class S, int CPL>
__global__ void __launch_bounds__(NW * 32, 4) tp_inner_spec_kernel(FusedArgs a) {
  constexpr int C = 32 * CPL, ROWF = S::DF * C;
  constexpr uint32_t ROWB = ROWF * sizeof(float);
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ uint64_t bars[2];
  Smem<S, CPL> sm(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int tb, te, rb, re;
  warp_ranges<S>(warp, tb, te, rb, re);
  float* wscale = sm.wbuf + warp * S::MAXT;
  for (int t = tb + lane; t < te; t += 32) wscale[t - tb] = __ldg(a.scale_k + t);
  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  cta_sync();

  const int64_t d0 = (int64_t)blockIdx.x * a.nodes_per_cta;
  const int64_t d1 = min(d0 + a.nodes_per_cta, a.n_out);
  const int64_t e0 = __ldg(a.ptr + d0), e1 = __ldg(a.ptr + d1);
  const int64_t nb = ceil_div(e1 - e0, STAGES);

  auto issue = [&](int64_t b) {
    if (tid == 0) {
      const int set = b & 1;
      const int64_t eb = e0 + b * STAGES;
      const int cnt = (int)min((int64_t)STAGES, e1 - eb);
      mbar_expect_tx(&bars[set], cnt * ROWB);
      for (int s = 0; s < cnt; ++s) {
        const int64_t row = a.fidx ? __ldg(a.fidx + eb + s) : eb + s;
        bulk_load(sm.xs + (set * STAGES + s) * ROWF, a.feat + row * ROWF, ROWB, &bars[set]);
      }
    }
  };

  float g[S::MAXR][CPL];
  int64_t d_cur = d0 - 1;
  int64_t boundary = e0;   // forces a load of G for the first node that has an edge
  auto next_node = [&]() {
    ++d_cur;
    boundary = __ldg(a.ptr + d_cur + 1);
    const float* gp = a.g + (d_cur * S::R + rb) * C + lane * CPL;
#pragma unroll
    for (int r = 0; r < S::MAXR; ++r) {
      if (r < re - rb) {
        if (CPL == 2) {
          const float2 v = __ldg(reinterpret_cast<const float2*>(gp + r * C));
          g[r][0] = v.x; g[r][CPL - 1] = v.y;
        } else {
          g[r][0] = __ldg(gp + r * C);
        }
      } else {
#pragma unroll
        for (int k = 0; k < CPL; ++k) g[r][k] = 0.f;
      }
    }
  };

  bool failed = false;
  if (nb > 0) issue(0);
  for (int64_t b = 0; b < nb; ++b) {
    if (b + 1 < nb) issue(b + 1);
    const int set = b & 1;
    if (!mbar_wait(&bars[set], (b >> 1) & 1)) { failed = true; break; }
    const int64_t eb = e0 + b * STAGES;
    const int cnt = (int)min((int64_t)STAGES, e1 - eb);
    for (int s = 0; s < cnt; ++s) {
      const int64_t e = eb + s;
      while (e >= boundary) next_node();
      float x[S::DF][CPL];
      const float* xr = sm.xs + (set * STAGES + s) * ROWF + lane * CPL;
#pragma unroll
      for (int m = 0; m < S::DF; ++m) {
        if (CPL == 2) {
          const float2 v = *reinterpret_cast<const float2*>(xr + m * C);
          x[m][0] = v.x; x[m][CPL - 1] = v.y;
        } else {
          x[m][0] = xr[m * C];
        }
      }
      float ay[S::DY];
#pragma unroll
      for (int k = 0; k < S::DY; ++k) ay[k] = 0.f;
      const float4* sc = reinterpret_cast<const float4*>(wscale);
      if (warp == 0) S::template inner_w0<CPL>(ay, x, g, sc);
      else if (warp == 1) S::template inner_w1<CPL>(ay, x, g, sc);
      else if (warp == 2) S::template inner_w2<CPL>(ay, x, g, sc);
      else S::template inner_w3<CPL>(ay, x, g, sc);
      float* rd = sm.red + ((set * STAGES + s) * NW + warp) * S::DY;
      warp_reduce_to_smem<S::DY>(ay, rd, lane);
    }
    cta_sync();
    // combine the four warps' partial sums of this batch; the other set is free until the next sync
    for (int q = tid; q < cnt * S::DY; q += NW * 32) {
      const int s = q / S::DY, k = q % S::DY;
      const float* rd = sm.red + ((set * STAGES + s) * NW) * S::DY + k;
      const float v = (rd[0] + rd[S::DY]) + (rd[2 * S::DY] + rd[3 * S::DY]);
      const int64_t e = eb + s;
      a.out[(a.yidx ? __ldg(a.yidx + e) : e) * S::DY + k] = v;
    }
  }
  if (failed) {
    if (tid == 0) atomicExch(a.status, 1);
    mbar_wait(&bars[0], 0);
    mbar_wait(&bars[1], 0);
  }
}

// ---- generic kernels ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) tp_segsum_generic_kernel(FusedArgs a) {
  const int64_t total = a.n_out * a.R * a.C;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int c = idx % a.C;
    const int r = (idx / a.C) % a.R;
    const int64_t d = idx / ((int64_t)a.C * a.R);
    const int64_t e0 = a.ptr ? __ldg(a.ptr + d) : d, e1 = a.ptr ? __ldg(a.ptr + d + 1) : d + 1;
    const int64_t t0 = __ldg(a.rowptr + r), t1 = __ldg(a.rowptr + r + 1);
    float acc = 0.f;
    for (int64_t e = e0; e < e1; ++e) {
      const float* xr = a.feat + (a.fidx ? __ldg(a.fidx + e) : e) * a.DF * a.C + c;
      const float* ye = a.y + (a.yidx ? __ldg(a.yidx + e) : e) * a.DY;
      for (int64_t t = t0; t < t1; ++t)
        acc = fmaf(__ldg(a.scale + t) * __ldg(ye + __ldg(a.my + t)), __ldg(xr + __ldg(a.mf + t) * a.C), acc);
    }
    a.out[idx] = acc;
  }
}

// one warp per edge; lane-private partial sums per y component live in shared memory
__global__ void __launch_bounds__(128) tp_inner_generic_kernel(FusedArgs a) {
  extern __shared__ float part[];   // [warps][DY][32]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  float* mine = part + warp * a.DY * 32;
  for (int64_t e = blockIdx.x * (int64_t)warps + warp; e < a.n_edges; e += (int64_t)gridDim.x * warps) {
    for (int k = 0; k < a.DY; ++k) mine[k * 32 + lane] = 0.f;
    const float* xr = a.feat + (a.fidx ? __ldg(a.fidx + e) : e) * a.DF * a.C;
    const float* gr = a.g + __ldg(a.enode + e) * a.R * a.C;
    for (int r = 0; r < a.R; ++r) {
      for (int64_t t = __ldg(a.rowptr + r); t < __ldg(a.rowptr + r + 1); ++t) {
        const float* xm = xr + __ldg(a.mf + t) * a.C;
        float p = 0.f;
        for (int c = lane; c < a.C; c += 32) p = fmaf(__ldg(xm + c), __ldg(gr + r * a.C + c), p);
        mine[__ldg(a.my + t) * 32 + lane] += __ldg(a.scale + t) * p;
      }
    }
    __syncwarp();
    float* o = a.out + (a.yidx ? __ldg(a.yidx + e) : e) * a.DY;
    for (int k = 0; k < a.DY; ++k) {
      float v = mine[k * 32 + lane];
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
      if (lane == 0) o[k] = v;
    }
    __syncwarp();
  }
}

// ---- dispatch ------------------------------------------------------------------------------------
template <class S, int CPL>
int launch_spec(bool inner, const FusedArgs& a, cudaStream_t s) {
  constexpr size_t bytes = spec_smem_bytes<S, CPL>();
  auto kern = inner ? tp_inner_spec_kernel<S, CPL> : tp_segsum_spec_kernel<S, CPL>;
  static bool configured[2] = {false, false};
  if (!configured[inner]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return fail(EQT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured[inner] = true;
  }
  const unsigned grid = (unsigned)ceil_div(a.n_out, a.nodes_per_cta);
  kern<<<grid, NW * 32, bytes, s>>>(a);
  return check_launch(inner ? "tp_inner_spec_kernel" : "tp_segsum_spec_kernel");
}

template <class S>
bool try_spec(uint64_t key, bool inner, const FusedArgs& a, cudaStream_t s, int& rc) {
  if (key != S::KEY || a.T != S::T || a.R != S::R || a.DF != S::DF || a.DY != S::DY) return false;
  if (a.C == 64) { rc = launch_spec<S, 2>(inner, a, s); return true; }
  if (a.C == 32) { rc = launch_spec<S, 1>(inner, a, s); return true; }
  return false;
}

int run(bool inner, const eqt_tp_table* tab, FusedArgs a, cudaStream_t s) {
  if (a.n_out == 0 || (inner && a.n_edges == 0)) return EQT_OK;
  if ((reinterpret_cast<uintptr_t>(a.feat) & 15u) == 0 && a.status && a.scale_k && a.my_k && (!inner || a.ptr)) {
    // nodes per CTA: keep every SM busy with several CTAs but amortise the pipeline prologue
    int64_t per = std::max<int64_t>(1, a.n_out / (148 * 16));
    const int64_t avg_deg = std::max<int64_t>(1, a.n_edges / std::max<int64_t>(1, a.n_out));
    per = std::min<int64_t>(per, std::max<int64_t>(1, 256 / avg_deg));
    a.nodes_per_cta = (int)per;
    int rc = EQT_OK;
#define EQT_TRY(SPEC) if (try_spec<specs::SPEC>(tab->structure_key, inner, a, s, rc)) return rc;
    EQT_FOR_EACH_SPEC(EQT_TRY)
#undef EQT_TRY
  }
  if (inner) {
    if (!a.enode) return fail(EQT_ERR_BAD_ARGUMENT, "edge_node is required by the table-driven kernel");
    const size_t bytes = sizeof(float) * 4 * a.DY * 32;
    if (bytes > 48 * 1024) return fail(EQT_ERR_UNSUPPORTED, "d_y = %d is too large for the table-driven kernel", a.DY);
    tp_inner_generic_kernel<<<flat_grid(a.n_edges, 4, 148 * 16), 128, bytes, s>>>(a);
    return check_launch("tp_inner_generic_kernel");
  }
  tp_segsum_generic_kernel<<<flat_grid(a.n_out * a.R * a.C, 256), 256, 0, s>>>(a);
  return check_launch("tp_segsum_generic_kernel");
}

int fill(const eqt_tp_table* tab, FusedArgs& a) {
  if (!tab || !tab->scale || !tab->m_feat || !tab->m_y || !tab->row_ptr) return fail(EQT_ERR_BAD_ARGUMENT, "incomplete table");
  if (tab->num_entries < 0 || tab->num_rows < 0 || tab->d_feat <= 0 || tab->d_y <= 0 || tab->d_y > 255)
    return fail(EQT_ERR_BAD_ARGUMENT, "bad table sizes");
  a.scale = tab->scale; a.mf = tab->m_feat; a.my = tab->m_y; a.rowptr = tab->row_ptr;
  a.scale_k = tab->scale_k; a.my_k = tab->m_y_k;
  a.T = tab->num_entries; a.R = tab->num_rows; a.DF = tab->d_feat; a.DY = tab->d_y;
  return EQT_OK;
}

}  // namespace
}  // namespace eqt

extern "C" int eqt_tp_cg_segment_sum(const eqt_tp_table* table, const float* feat, const int64_t* feat_index,
                                     const float* y, const int64_t* y_index, const int64_t* seg_ptr, float* out,
                                     int64_t num_out, int64_t num_edges, int32_t channels, int32_t* status,
                                     void* stream) {
  using namespace eqt;
  FusedArgs a{};
  if (int rc = fill(table, a)) return rc;
  if (num_out < 0 || num_edges < 0 || channels <= 0) return fail(EQT_ERR_BAD_ARGUMENT, "bad sizes");
  if ((num_out > 0 && (!feat || !out)) || (num_edges > 0 && !y)) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  if (!seg_ptr && num_out != num_edges) return fail(EQT_ERR_BAD_ARGUMENT, "without seg_ptr there is one output per edge");
  a.feat = feat; a.fidx = feat_index; a.y = y; a.yidx = y_index; a.ptr = seg_ptr; a.out = out;
  a.n_out = num_out; a.n_edges = num_edges; a.C = channels; a.status = status;
  return run(false, table, a, static_cast<cudaStream_t>(stream));
}

extern "C" int eqt_tp_cg_inner(const eqt_tp_table* table, const float* feat, const int64_t* feat_index,
                               const float* g, const int64_t* seg_ptr, const int64_t* edge_node,
                               const int64_t* y_index, float* grad_y, int64_t num_nodes, int64_t num_edges,
                               int32_t channels, int32_t* status, void* stream) {
  using namespace eqt;
  FusedArgs a{};
  if (int rc = fill(table, a)) return rc;
  if (num_nodes < 0 || num_edges < 0 || channels <= 0) return fail(EQT_ERR_BAD_ARGUMENT, "bad sizes");
  if (num_edges > 0 && (!feat || !g || !grad_y || (!seg_ptr && !edge_node))) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  a.feat = feat; a.fidx = feat_index; a.g = g; a.ptr = seg_ptr; a.enode = edge_node; a.yidx = y_index; a.out = grad_y;
  a.n_out = num_nodes; a.n_edges = num_edges; a.C = channels; a.status = status;
  return run(true, table, a, static_cast<cudaStream_t>(stream));
}
