// Wigner-D matrices from ZYZ Euler angles and their application to features.
//
//   D(alpha, beta, gamma) = Z(alpha) J Z(beta) J Z(gamma)        per irrep block of degree l, n = 2l + 1,
//
// with Z(a) the real-basis z-rotation  x'_m = cos(m a) x_m - sign(m) sin(|m| a) x_{-m}  and J the constant,
// symmetric, involutive block that exchanges the y and z axes.  The reference builds D by pushing the identity
// through five sparse passes over a dense (N, dim, dim) tensor and differentiates through all of them; here one
// kernel writes D directly from the angles and one kernel turns grad_D into the three angle gradients.
//
// The middle factor is a trigonometric polynomial in beta with constant coefficients,
//
//   d(beta) = J Z(beta) J = sum_{k=0..l}  A_k cos(k beta) + B_k sin(k beta),
//   A_k[a][b] = J[a][k] J[k][b] + J[a][-k] J[-k][b]      (A_0 = J[a][0] J[0][b]),
//   B_k[a][b] = -J[a][k] J[-k][b] + J[a][-k] J[k][b],
//
// (indices are m values), so an element D[p][q] needs d at the four positions (+-p, +-q) and a few sines and
// cosines:  T[a][q] = d[a][q] cos(q g) + sign(q) d[a][-q] sin(|q| g),   D[p][q] = cos(p a) T[p][q] - sign(p) sin(|p| a) T[-p][q].
// The coefficient tables (5208 floats for l = 0..6) live in shared memory.
//
// Also here: the dense rotation  out[n] = D[n] x[n]  (and with D transposed) and its gradient with respect to D,
// as shared-memory tiled kernels (a 49 x 49 matrix per sample is too small for a library GEMM to pay off and the
// operands are read exactly once).
#include <algorithm>

#include "common.cuh"

namespace eqt {
namespace {

constexpr int WIG_EPB = 4;          // samples per CTA iteration of the forward kernel
constexpr int WIG_MAX_L = 7;

struct WigArgs {
  const void* coef;             // per block: (l + 1) x n x n x 2 values [k][a][b][A, B]
  const int32_t* comp;          // (dim, 4): block start, l, coefficient offset (in values), m
  const void* alpha;
  const void* beta;
  const void* gamma;
  void* d;                      // forward: out (N, dim, dim); backward: grad_d
  void* ga;
  void* gb;
  void* gc;
  int64_t n;
  int dim, max_l, coef_count;
  int block_elems;              // capacity of the forward kernel's in-block element list (dim * dim always suffices)
};

template <typename T> __device__ __forceinline__ void sincos_t(T x, T* s, T* c);
template <> __device__ __forceinline__ void sincos_t<float>(float x, float* s, float* c) { sincosf(x, s, c); }
template <> __device__ __forceinline__ void sincos_t<double>(double x, double* s, double* c) { sincos(x, s, c); }

// Trig table of one sample: tr[which][k] = (cos(k angle), sin(k angle)), which = 0 alpha, 1 beta, 2 gamma; the product
// k * angle is formed in the working precision first, as the reference does.
template <typename T>
__device__ __forceinline__ void fill_trig(T* tr, int L1, int which, int k, T angle) {
  T s, c;
  sincos_t<T>(angle * T(k), &s, &c);
  tr[(which * L1 + k) * 2] = c;
  tr[(which * L1 + k) * 2 + 1] = s;
}

// One element of a block of degree l at m values (p, q).  coef points at the block's table, tr at the sample's trig
// table.  With GRAD the derivatives with respect to the three angles are produced too.
template <typename T, bool GRAD>
__device__ __forceinline__ void wigner_element(const T* coef, const T* tr, int L1, int l, int p, int q, T& D, T& Da, T& Db, T& Dg) {
  const int n = 2 * l + 1, nn2 = n * n * 2;
  const T* tb = tr + L1 * 2;                    // beta
  const int ap = p < 0 ? -p : p, aq = q < 0 ? -q : q;
  // d and d' = dd/dbeta at (a, b), a in {p, -p}, b in {q, -q}
  T dv[2][2], dd[2][2];
#pragma unroll
  for (int ia = 0; ia < 2; ++ia) {
#pragma unroll
    for (int ib = 0; ib < 2; ++ib) {
      dv[ia][ib] = T(0);
      dd[ia][ib] = T(0);
      if ((ia == 1 && p == 0) || (ib == 1 && q == 0)) continue;
      const int a = ia ? -p : p, b = ib ? -q : q;
      const T* cf = coef + ((a + l) * n + (b + l)) * 2;
      T acc = T(0), der = T(0);
      for (int k = 0; k <= l; ++k) {
        const T A = cf[k * nn2], B = cf[k * nn2 + 1], ck = tb[2 * k], sk = tb[2 * k + 1];
        acc += A * ck + B * sk;
        if (GRAD) der += T(k) * (B * ck - A * sk);
      }
      dv[ia][ib] = acc;
      dd[ia][ib] = der;
    }
  }
  const T* tg = tr + 2 * L1 * 2;                // gamma
  const T cq = tg[2 * aq], sq = (q > 0 ? T(1) : q < 0 ? T(-1) : T(0)) * tg[2 * aq + 1];
  const T cp = tr[2 * ap], sp = (p > 0 ? T(1) : p < 0 ? T(-1) : T(0)) * tr[2 * ap + 1];
  // T[a][q] for a = p (row 0) and a = -p (row 1)
  const T t0 = dv[0][0] * cq + dv[0][1] * sq, t1 = dv[1][0] * cq + dv[1][1] * sq;
  D = cp * t0 - sp * t1;
  if (GRAD) {
    const T tb0 = dd[0][0] * cq + dd[0][1] * sq, tb1 = dd[1][0] * cq + dd[1][1] * sq;
    // d/dgamma: cos(q g) -> -|q| sin(|q| g);  sign(q) sin(|q| g) -> q cos(q g)
    const T dcq = -T(aq) * tg[2 * aq + 1], dsq = T(q) * tg[2 * aq];
    const T tg0 = dv[0][0] * dcq + dv[0][1] * dsq, tg1 = dv[1][0] * dcq + dv[1][1] * dsq;
    const T dcp = -T(ap) * tr[2 * ap + 1], dsp = T(p) * tr[2 * ap];
    Da = dcp * t0 - dsp * t1;
    Db = cp * tb0 - sp * tb1;
    Dg = cp * tg0 - sp * tg1;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) wigner_d_forward_kernel(WigArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* coef = reinterpret_cast<T*>(smem_raw);
  T* tr = coef + a.coef_count;                                  // [WIG_EPB][3][L1][2]
  // in-block elements of the dim x dim matrix: position and (coefficient offset << 12) | (l << 8) | ((p + l) << 4) | (q + l);
  // `img` holds one sample's matrix: zeros outside the blocks (written once), the blocks rewritten per sample, so that
  // only block elements cost arithmetic and every sample leaves as one linear, coalesced copy
  int32_t* elem = reinterpret_cast<int32_t*>(tr + WIG_EPB * 3 * (a.max_l + 1) * 2);     // [count][2]
  const int L1 = a.max_l + 1, dim = a.dim, dd = dim * dim;
  T* img = reinterpret_cast<T*>(elem + 2 * a.block_elems);
  __shared__ int count_s;
  if (threadIdx.x == 0) count_s = 0;
  for (int i = threadIdx.x; i < a.coef_count; i += blockDim.x) coef[i] = static_cast<const T*>(a.coef)[i];
  for (int i = threadIdx.x; i < dd; i += blockDim.x) img[i] = T(0);
  __syncthreads();
  for (int i = threadIdx.x; i < dd; i += blockDim.x) {
    const int P = i / dim, Q = i % dim;
    const int32_t* cp = a.comp + 4 * P;
    const int32_t* cq = a.comp + 4 * Q;
    if (__ldg(cp) == __ldg(cq)) {
      const int l = __ldg(cp + 1);
      const int slot = atomicAdd(&count_s, 1);      // any order: every element is written by exactly one thread per sample
      elem[2 * slot] = i;
      elem[2 * slot + 1] = (__ldg(cp + 2) << 12) | (l << 8) | ((__ldg(cp + 3) + l) << 4) | (__ldg(cq + 3) + l);
    }
  }
  const T* angles[3] = {static_cast<const T*>(a.alpha), static_cast<const T*>(a.beta), static_cast<const T*>(a.gamma)};
  T* out = static_cast<T*>(a.d);
  for (int64_t s0 = (int64_t)blockIdx.x * WIG_EPB; s0 < a.n; s0 += (int64_t)gridDim.x * WIG_EPB) {
    __syncthreads();                                            // tables loaded / previous samples done with the trig table
    const int ns = (int)min((int64_t)WIG_EPB, a.n - s0);
    for (int i = threadIdx.x; i < ns * 3 * L1; i += blockDim.x) {
      const int s = i / (3 * L1), r = i % (3 * L1), which = r / L1, k = r % L1;
      fill_trig<T>(tr + s * 3 * L1 * 2, L1, which, k, angles[which][s0 + s]);
    }
    __syncthreads();
    const int count = count_s;
    for (int s = 0; s < ns; ++s) {
      for (int e = threadIdx.x; e < count; e += blockDim.x) {
        const int32_t code = elem[2 * e + 1];
        const int l = (code >> 8) & 15;
        T v, u0, u1, u2;
        wigner_element<T, false>(coef + (code >> 12), tr + s * 3 * L1 * 2, L1, l, ((code >> 4) & 15) - l, (code & 15) - l, v, u0, u1, u2);
        img[elem[2 * e]] = v;
      }
      __syncthreads();
      T* o = out + (s0 + s) * dd;
      for (int r = threadIdx.x; r < dd; r += blockDim.x) o[r] = img[r];
      __syncthreads();
    }
  }
}

// one warp per sample; the lanes stride over the elements of every block and the three sums are reduced with shuffles
template <typename T>
__global__ void __launch_bounds__(256) wigner_d_backward_kernel(WigArgs a, int num_blocks, const int32_t* __restrict__ blocks) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* coef = reinterpret_cast<T*>(smem_raw);
  const int L1 = a.max_l + 1, dim = a.dim, warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  T* tr = coef + a.coef_count + warp * 3 * L1 * 2;
  for (int i = threadIdx.x; i < a.coef_count; i += blockDim.x) coef[i] = static_cast<const T*>(a.coef)[i];
  __syncthreads();
  const T* angles[3] = {static_cast<const T*>(a.alpha), static_cast<const T*>(a.beta), static_cast<const T*>(a.gamma)};
  const T* gd = static_cast<const T*>(a.d);
  for (int64_t s = (int64_t)blockIdx.x * warps + warp; s < a.n; s += (int64_t)gridDim.x * warps) {
    __syncwarp();
    for (int i = lane; i < 3 * L1; i += 32) fill_trig<T>(tr, L1, i / L1, i % L1, angles[i / L1][s]);
    __syncwarp();
    T sa = T(0), sb = T(0), sg = T(0);
    for (int b = 0; b < num_blocks; ++b) {
      const int start = __ldg(blocks + 3 * b), l = __ldg(blocks + 3 * b + 1), off = __ldg(blocks + 3 * b + 2), n = 2 * l + 1;
      for (int i = lane; i < n * n; i += 32) {
        const int pi = i / n, qi = i % n;
        T D, Da, Db, Dg;
        wigner_element<T, true>(coef + off, tr, L1, l, pi - l, qi - l, D, Da, Db, Dg);
        const T g = gd[(s * dim + start + pi) * dim + start + qi];
        sa += g * Da;
        sb += g * Db;
        sg += g * Dg;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sa += __shfl_xor_sync(0xffffffffu, sa, o);
      sb += __shfl_xor_sync(0xffffffffu, sb, o);
      sg += __shfl_xor_sync(0xffffffffu, sg, o);
    }
    if (lane == 0) {
      static_cast<T*>(a.ga)[s] = sa;
      static_cast<T*>(a.gb)[s] = sb;
      static_cast<T*>(a.gc)[s] = sg;
    }
  }
}

// ---- dense rotation: out[n, i, c] = sum_j M[n, i, j] x[n, j, c]   (transposed: M[n, j, i]) ---------------------
// One CTA per sample: M (dim x dim) and x (dim x C) are staged in shared memory, M with the contraction index
// outermost, so that a thread producing a 4 x 4 tile (4 rows, 4 channels) needs two 16-byte loads per contraction
// step.  Rows and channels are padded to multiples of four inside shared memory only.
// Asynchronous global -> shared copies of one element (4 or 8 bytes) or of 16 bytes.  Staging a sample through
// registers (load, dependent store, next load) leaves one load in flight per thread: 30 elements per thread at the
// latency of HBM each made these kernels latency bound at a fifth of the bandwidth; cp.async keeps them all in flight.
template <int BYTES>
__device__ __forceinline__ void cp_async(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  if (BYTES == 16)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(s), "l"(gmem), "n"(BYTES) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <typename T> struct alignas(16) Vec4 { T v[4]; };

template <typename T>
__global__ void __launch_bounds__(128) dense_rotation_kernel(const T* __restrict__ mat, const T* __restrict__ x, T* __restrict__ out,
                                                             int64_t n, int dim, int c, int transposed,
                                                             const int32_t* __restrict__ row_range) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int dim4 = (dim + 3) & ~3, c4 = (c + 3) & ~3;
  T* ms = reinterpret_cast<T*>(smem_raw);        // [j][i padded to dim4]: ms[j * dim4 + i] = M[i][j] (or M[j][i] when transposed)
  T* xs = ms + dim * dim4;                       // [j][c padded to c4]
  for (int i = threadIdx.x; i < dim * dim4; i += blockDim.x) ms[i] = T(0);
  for (int i = threadIdx.x; i < dim * c4; i += blockDim.x) xs[i] = T(0);
  const int rgroups = dim4 / 4, cgroups = c4 / 4;
  for (int64_t s = blockIdx.x; s < n; s += gridDim.x) {
    __syncthreads();
    const T* m = mat + s * dim * dim;
    // row_range (block-diagonal matrices): only columns [lo, hi) of a row are read, the rest of `ms` keeps its zeros
    for (int r = threadIdx.x / 32; r < dim; r += blockDim.x / 32)
      for (int q = (row_range ? __ldg(row_range + 2 * r) : 0) + threadIdx.x % 32, qe = row_range ? __ldg(row_range + 2 * r + 1) : dim;
           q < qe; q += 32)                                        // element M[r][q]; the contraction index is the row when transposed
        cp_async<sizeof(T)>(transposed ? ms + r * dim4 + q : ms + q * dim4 + r, m + r * dim + q);
    const T* xin = x + s * dim * c;
    if (c == c4 && (reinterpret_cast<uintptr_t>(xin) & 15u) == 0) {
      constexpr int PER = 16 / sizeof(T);
      for (int i = threadIdx.x; i < dim * c / PER; i += blockDim.x) cp_async<16>(xs + i * PER, xin + i * PER);
    } else {
      for (int r = threadIdx.x / 32; r < dim; r += blockDim.x / 32)
        for (int q = threadIdx.x % 32; q < c; q += 32) cp_async<sizeof(T)>(xs + r * c4 + q, xin + r * c + q);
    }
    cp_async_wait_all();
    __syncthreads();
    T* o = out + s * dim * c;
    for (int i = threadIdx.x; i < rgroups * cgroups; i += blockDim.x) {
      const int ch = (i % cgroups) * 4, r0 = (i / cgroups) * 4;
      T acc[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int w = 0; w < 4; ++w) acc[u][w] = T(0);
      int jlo = 0, jhi = dim;
      if (row_range) {                             // contraction range of the tile's rows (the blocks are square)
        const int r1 = min(r0 + 3, dim - 1);
        jlo = __ldg(row_range + 2 * r0);
        jhi = __ldg(row_range + 2 * r1 + 1);
      }
      for (int j = jlo; j < jhi; ++j) {
        const Vec4<T> xv = *reinterpret_cast<const Vec4<T>*>(xs + j * c4 + ch);
        const Vec4<T> mv = *reinterpret_cast<const Vec4<T>*>(ms + j * dim4 + r0);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int w = 0; w < 4; ++w) acc[u][w] += mv.v[u] * xv.v[w];
      }
      const bool vec = (c & 3) == 0 && (reinterpret_cast<uintptr_t>(o) & 15u) == 0;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (r0 + u >= dim) break;
        if (vec) {
          Vec4<T> v;
#pragma unroll
          for (int w = 0; w < 4; ++w) v.v[w] = acc[u][w];
          *reinterpret_cast<Vec4<T>*>(o + (r0 + u) * c + ch) = v;
        } else {
#pragma unroll
          for (int w = 0; w < 4; ++w)
            if (ch + w < c) o[(r0 + u) * c + ch + w] = acc[u][w];
        }
      }
    }
  }
}

// grad_M[n, i, j] = sum_c g[n, i, c] x[n, j, c]: g and x are staged channel-major ([c][i]), a thread produces a
// 4 x 4 tile of grad_M from two 16-byte loads per channel
template <typename T>
__global__ void __launch_bounds__(256) dense_rotation_grad_matrix_kernel(const T* __restrict__ g, const T* __restrict__ x, T* __restrict__ gm,
                                                                         int64_t n, int dim, int c,
                                                                         const int32_t* __restrict__ row_range) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int dim4 = (dim + 3) & ~3;
  T* gs = reinterpret_cast<T*>(smem_raw);        // [c][i padded to dim4]
  T* xs = gs + c * dim4;
  T* img = xs + c * dim4;                        // [dim][dim] result of the current sample
  for (int i = threadIdx.x; i < 2 * c * dim4; i += blockDim.x) gs[i] = T(0);
  const int groups = dim4 / 4;
  for (int64_t s = blockIdx.x; s < n; s += gridDim.x) {
    __syncthreads();
    // consecutive threads read consecutive channels of one row (coalesced); the transposing store is padded by the
    // row pitch dim4 (odd multiples of four words spread over the banks well enough for this one pass)
    const T* gsrc = g + s * dim * c;
    const T* xsrc = x + s * dim * c;
    bool staged = false;
    if constexpr (sizeof(T) == 4) {
     if ((c & 3) == 0 && ((reinterpret_cast<uintptr_t>(gsrc) | reinterpret_cast<uintptr_t>(xsrc)) & 15u) == 0) {
      staged = true;
      // 16-byte loads of both operands first (all in flight), then the transposing scalar stores: element-wise
      // asynchronous copies to transposed addresses ran at about one element per cycle and SM
      const int quads = dim * c / 4;
      for (int i0 = threadIdx.x; i0 < quads; i0 += 2 * blockDim.x) {
        float4 gv[2], xv[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int i = i0 + u * blockDim.x;
          if (i < quads) {
            gv[u] = __ldg(reinterpret_cast<const float4*>(gsrc) + i);
            xv[u] = __ldg(reinterpret_cast<const float4*>(xsrc) + i);
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int i = i0 + u * blockDim.x;
          if (i < quads) {
            const int r = (i * 4) / c, k = (i * 4) % c;
            const float ga[4] = {gv[u].x, gv[u].y, gv[u].z, gv[u].w}, xa[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              gs[(k + w) * dim4 + r] = ga[w];
              xs[(k + w) * dim4 + r] = xa[w];
            }
          }
        }
      }
     }
    }
    if (!staged) {
      for (int r = threadIdx.x / 32; r < dim; r += blockDim.x / 32)
        for (int k = threadIdx.x % 32; k < c; k += 32) {
          cp_async<sizeof(T)>(gs + k * dim4 + r, gsrc + r * c + k);
          cp_async<sizeof(T)>(xs + k * dim4 + r, xsrc + r * c + k);
        }
      cp_async_wait_all();
    }
    __syncthreads();
    T* o = gm + s * dim * dim;
    for (int i = threadIdx.x; i < groups * groups; i += blockDim.x) {
      const int q0 = (i % groups) * 4, p0 = (i / groups) * 4;
      T acc[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int w = 0; w < 4; ++w) acc[u][w] = T(0);
      // block-diagonal matrices: a tile outside every block of its rows is written as zeros without the products
      bool inside = true;
      if (row_range) {
        const int p1 = min(p0 + 3, dim - 1);
        inside = p0 < dim && q0 < __ldg(row_range + 2 * p1 + 1) && q0 + 4 > __ldg(row_range + 2 * p0);
      }
      for (int k = 0; k < (inside ? c : 0); ++k) {
        const Vec4<T> gv = *reinterpret_cast<const Vec4<T>*>(gs + k * dim4 + p0);
        const Vec4<T> xv = *reinterpret_cast<const Vec4<T>*>(xs + k * dim4 + q0);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int w = 0; w < 4; ++w) acc[u][w] += gv.v[u] * xv.v[w];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int w = 0; w < 4; ++w)
          if (p0 + u < dim && q0 + w < dim) {
            // inside a straddling tile, entries outside the row's own block are zero as well
            const bool keep = !row_range || (q0 + w >= __ldg(row_range + 2 * (p0 + u)) && q0 + w < __ldg(row_range + 2 * (p0 + u) + 1));
            img[(p0 + u) * dim + q0 + w] = keep ? acc[u][w] : T(0);
          }
    }
    // the sample's matrix is contiguous in memory: it leaves as one linear copy (the tiles' own 4 x 4 patches would be
    // sixteen strided scalar stores per thread)
    __syncthreads();
    for (int i = threadIdx.x; i < dim * dim; i += blockDim.x) o[i] = img[i];
  }
}

int wig_check(const eqt_wigner_table* t, int32_t dtype) {
  if (!t || !t->coef || !t->comp || !t->blocks) return fail(EQT_ERR_BAD_ARGUMENT, "incomplete Wigner table");
  if (t->dim <= 0 || t->num_blocks <= 0 || t->max_l < 0 || t->max_l > WIG_MAX_L)
    return fail(EQT_ERR_UNSUPPORTED, "Wigner kernels take degrees up to %d", WIG_MAX_L);
  if (dtype != EQT_F32 && dtype != EQT_F64) return fail(EQT_ERR_UNSUPPORTED, "float32 or float64 only");
  return EQT_OK;
}

template <typename T>
int wig_launch(bool backward, const eqt_wigner_table* t, WigArgs a, cudaStream_t st) {
  const int L1 = t->max_l + 1;
  if (!backward) {
    a.block_elems = t->dim * t->dim;
    const size_t bytes = sizeof(T) * ((size_t)t->coef_count + WIG_EPB * 3 * L1 * 2 + (size_t)t->dim * t->dim) +
                         sizeof(int32_t) * 2 * a.block_elems;
    if (t->max_l > 7 || t->coef_count >= (1 << 19)) return fail(EQT_ERR_UNSUPPORTED, "element codes hold degrees up to 7");
    if (bytes > 200 * 1024) return fail(EQT_ERR_UNSUPPORTED, "Wigner coefficient table too large for shared memory");
    cudaError_t e = cudaFuncSetAttribute(wigner_d_forward_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return fail(EQT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    // one resident wave (the per-CTA tables make a second, partial wave expensive)
    int per_sm = 1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, wigner_d_forward_kernel<T>, 256, bytes) != cudaSuccess || per_sm < 1)
      per_sm = 1;
    const unsigned grid = (unsigned)std::min<int64_t>(ceil_div(a.n, WIG_EPB), (int64_t)sm_count() * per_sm);
    wigner_d_forward_kernel<T><<<grid, 256, bytes, st>>>(a);
    return check_launch("wigner_d_forward_kernel");
  }
  const size_t bytes = sizeof(T) * ((size_t)t->coef_count + 8 * 3 * L1 * 2);
  if (bytes > 200 * 1024) return fail(EQT_ERR_UNSUPPORTED, "Wigner coefficient table too large for shared memory");
  cudaError_t e = cudaFuncSetAttribute(wigner_d_backward_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) return fail(EQT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  int per_sm = 1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, wigner_d_backward_kernel<T>, 256, bytes) != cudaSuccess || per_sm < 1)
    per_sm = 1;
  const unsigned grid = (unsigned)std::min<int64_t>(ceil_div(a.n, 8), (int64_t)sm_count() * per_sm);
  wigner_d_backward_kernel<T><<<grid, 256, bytes, st>>>(a, t->num_blocks, t->blocks);
  return check_launch("wigner_d_backward_kernel");
}

}  // namespace
}  // namespace eqt

extern "C" int eqt_wigner_d_forward(const eqt_wigner_table* table, const void* alpha, const void* beta, const void* gamma,
                                    void* d, int64_t n, int32_t dtype, void* stream) {
  using namespace eqt;
  if (int rc = wig_check(table, dtype)) return rc;
  if (n < 0) return fail(EQT_ERR_BAD_ARGUMENT, "bad sizes");
  if (n == 0) return EQT_OK;
  if (!alpha || !beta || !gamma || !d) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  WigArgs a{};
  a.coef = table->coef; a.comp = table->comp; a.alpha = alpha; a.beta = beta; a.gamma = gamma; a.d = d; a.n = n;
  a.dim = table->dim; a.max_l = table->max_l; a.coef_count = table->coef_count;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == EQT_F32 ? wig_launch<float>(false, table, a, st) : wig_launch<double>(false, table, a, st);
}

extern "C" int eqt_wigner_d_backward(const eqt_wigner_table* table, const void* alpha, const void* beta, const void* gamma,
                                     const void* grad_d, void* grad_alpha, void* grad_beta, void* grad_gamma, int64_t n,
                                     int32_t dtype, void* stream) {
  using namespace eqt;
  if (int rc = wig_check(table, dtype)) return rc;
  if (n < 0) return fail(EQT_ERR_BAD_ARGUMENT, "bad sizes");
  if (n == 0) return EQT_OK;
  if (!alpha || !beta || !gamma || !grad_d || !grad_alpha || !grad_beta || !grad_gamma) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  WigArgs a{};
  a.coef = table->coef; a.comp = table->comp; a.alpha = alpha; a.beta = beta; a.gamma = gamma;
  a.d = const_cast<void*>(grad_d); a.ga = grad_alpha; a.gb = grad_beta; a.gc = grad_gamma; a.n = n;
  a.dim = table->dim; a.max_l = table->max_l; a.coef_count = table->coef_count;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == EQT_F32 ? wig_launch<float>(true, table, a, st) : wig_launch<double>(true, table, a, st);
}

extern "C" int eqt_dense_rotation(const void* matrix, const void* x, void* out, int64_t n, int32_t dim, int32_t channels,
                                  int32_t transposed, const int32_t* row_range, int32_t dtype, void* stream) {
  using namespace eqt;
  if (n < 0 || dim <= 0 || channels <= 0) return fail(EQT_ERR_BAD_ARGUMENT, "bad sizes");
  if (dtype != EQT_F32 && dtype != EQT_F64) return fail(EQT_ERR_UNSUPPORTED, "float32 or float64 only");
  if (n == 0) return EQT_OK;
  if (!matrix || !x || !out) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  const size_t es = dtype == EQT_F32 ? 4 : 8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t bytes = es * ((size_t)dim * ((dim + 3) & ~3) + (size_t)dim * ((channels + 3) & ~3));
  if (bytes > 200 * 1024) return fail(EQT_ERR_UNSUPPORTED, "matrix and features of one sample do not fit shared memory");
  // one resident wave: samples are strided over the CTAs, and a second, partial wave would run at a fraction of the occupancy
  auto wave = [&](auto kernel, int threads) {
    int per_sm = 1;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, bytes) != cudaSuccess || per_sm < 1) per_sm = 1;
    return (unsigned)std::min<int64_t>(n, (int64_t)sm_count() * per_sm);
  };
  if (dtype == EQT_F32) {
    const unsigned grid = wave(dense_rotation_kernel<float>, 128);
    dense_rotation_kernel<float><<<grid, 128, bytes, st>>>(static_cast<const float*>(matrix), static_cast<const float*>(x),
                                                            static_cast<float*>(out), n, dim, channels, transposed, row_range);
  } else {
    const unsigned grid = wave(dense_rotation_kernel<double>, 128);
    dense_rotation_kernel<double><<<grid, 128, bytes, st>>>(static_cast<const double*>(matrix), static_cast<const double*>(x),
                                                             static_cast<double*>(out), n, dim, channels, transposed, row_range);
  }
  return check_launch("dense_rotation_kernel");
}

extern "C" int eqt_dense_rotation_grad_matrix(const void* grad_out, const void* x, void* grad_matrix, int64_t n, int32_t dim,
                                              int32_t channels, const int32_t* row_range, int32_t dtype, void* stream) {
  using namespace eqt;
  if (n < 0 || dim <= 0 || channels <= 0) return fail(EQT_ERR_BAD_ARGUMENT, "bad sizes");
  if (dtype != EQT_F32 && dtype != EQT_F64) return fail(EQT_ERR_UNSUPPORTED, "float32 or float64 only");
  if (n == 0) return EQT_OK;
  if (!grad_out || !x || !grad_matrix) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  const size_t es = dtype == EQT_F32 ? 4 : 8;
  const size_t bytes = es * (2 * (size_t)channels * ((dim + 3) & ~3) + (size_t)dim * dim);
  if (bytes > 200 * 1024) return fail(EQT_ERR_UNSUPPORTED, "features of one sample do not fit shared memory");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto wave = [&](auto kernel, int threads) {
    int per_sm = 1;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, bytes) != cudaSuccess || per_sm < 1) per_sm = 1;
    return (unsigned)std::min<int64_t>(n, (int64_t)sm_count() * per_sm);
  };
  if (dtype == EQT_F32) {
    const unsigned grid = wave(dense_rotation_grad_matrix_kernel<float>, 256);
    dense_rotation_grad_matrix_kernel<float><<<grid, 256, bytes, st>>>(static_cast<const float*>(grad_out), static_cast<const float*>(x),
                                                                        static_cast<float*>(grad_matrix), n, dim, channels, row_range);
  } else {
    const unsigned grid = wave(dense_rotation_grad_matrix_kernel<double>, 256);
    dense_rotation_grad_matrix_kernel<double><<<grid, 256, bytes, st>>>(static_cast<const double*>(grad_out), static_cast<const double*>(x),
                                                                         static_cast<double*>(grad_matrix), n, dim, channels, row_range);
  }
  return check_launch("dense_rotation_grad_matrix_kernel");
}
