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
//  * "spec": for index structures unrolled at build time (generated/tp_specs.inc).  The sum over
//    the edges of a node commutes with the CG contraction, so per edge only the dense outer
//    product Q[m_y, m_feat] += y_e[m_y] x_e[m_feat] is accumulated (234 of the 256 cells are used
//    at l_max = 3) and the 353-entry sparse contraction runs once per node.  One CTA walks a
//    contiguous range of destination nodes; feature rows of the next four edges are fetched with
//    bulk asynchronous copies (cp.async.bulk + mbarrier, double buffered) while the current four
//    are consumed.  A warp handles 32 channels (one per lane) and one half of the cells, chosen
//    so that every intermediate row is produced by exactly one warp from its own registers.  No
//    atomics: the edges of a node are consecutive.  The adjoint runs the same scheme backwards:
//    H[cell] = sum_t scale[t] G_d[row(t)] once per node, then a dense dot product per edge.
//  * "generic": table-driven, one thread per output element; any structure, any channel count.
#include <algorithm>

#include "common.cuh"

namespace eqt {
namespace specs {
#include "generated/tp_specs.inc"
}  // namespace specs

namespace {

constexpr int STAGES = 4;   // edges per batch
constexpr int WAIT_SPINS = 1 << 22;

struct FusedArgs {
  const float* feat;        // (rows, DF, C)
  const int64_t* fidx;      // (E) feature row of each edge, or NULL (= e)
  const float* y;           // (Ey, DY)
  const int64_t* yidx;      // (E) row of y (and of grad_y) of each edge, or NULL (= e)
  const int64_t* ptr;       // (N + 1) CSR of edges per output node, or NULL (one edge per output)
  const int64_t* enode;     // (E) node of each edge (generic inner kernel only)
  const float* scale;       // (T)
  const float* scale_o;     // scales in the unrolled kernels' role order (zero padded), or NULL
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
__device__ __forceinline__ void cp_async_4(void* dst_smem, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_addr(dst_smem)), "l"(src) : "memory");
}
// one arrival (already part of the barrier's init count) once this thread's earlier cp.async have landed
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// Shared memory of the spec kernels for a CTA of NWARP warps and a ring of NS batches.
template <class S, int CQ>
struct Smem {
  static constexpr int C = 32 * CQ, NWARP = 2 * CQ, ROWF = S::DF * C;
  static constexpr int NS = 6;    // batches in flight (ring of STAGES-edge sets); 4 KB rows at C = 64: 96 KB per CTA
  float* xs;      // [NS][STAGES][DF * C] gathered feature rows
  float* ys;      // [NS][STAGES][DY] harmonics rows of the batch (segment sum)
  float* ssc;     // [OT2] scales in role order
  float* red;     // [2][STAGES][NWARP][DY] per-warp partial grad_y, two sets (adjoint)
  __device__ explicit Smem(unsigned char* base) {
    xs = reinterpret_cast<float*>(base);
    ys = xs + NS * STAGES * ROWF;
    ssc = ys + NS * STAGES * S::DY;
    red = ssc + S::OT2;
  }
  static constexpr size_t bytes() {
    return sizeof(float) * (NS * STAGES * ROWF + NS * STAGES * S::DY + S::OT2 + 2 * STAGES * NWARP * S::DY) + 64;
  }
};

// Ring of edge batches filled NS - 1 batches ahead of their use by warp 0: feature rows by bulk copies
// (lane s copies the row of edge s), harmonics elements by 4-byte cp.async, both completing on the
// batch's mbarrier (1 arrival for the expected bytes + 1 per lane of warp 0 for its cp.async).  The
// gather indices of a batch are read one iteration before they are needed, so no global-memory
// latency sits between two batches.
template <class S, int CQ, bool WITH_Y>
struct EdgeRing {
  using SM = Smem<S, CQ>;
  static constexpr int NS = SM::NS, ROWF = SM::ROWF;
  static constexpr uint32_t ROWB = ROWF * sizeof(float);
  const FusedArgs& a;
  SM& sm;
  uint64_t* bars;
  int64_t e0, e1, nb;
  int warp, lane;
  int64_t fi = 0, yi = 0;   // warp 0, lane s: indices of edge s of the next batch to issue

  __device__ EdgeRing(const FusedArgs& a_, SM& sm_, uint64_t* bars_, int64_t e0_, int64_t e1_, int warp_, int lane_)
      : a(a_), sm(sm_), bars(bars_), e0(e0_), e1(e1_), nb(ceil_div(e1_ - e0_, STAGES)), warp(warp_), lane(lane_) {}

  __device__ void load_idx(int64_t bb) {
    const int64_t e = e0 + bb * STAGES + lane;
    if (lane < STAGES && e < e1) {
      fi = a.fidx ? __ldg(a.fidx + e) : e;
      if (WITH_Y) yi = a.yidx ? __ldg(a.yidx + e) : e;
    }
  }
  __device__ void issue(int64_t bb) {   // whole warp 0; indices of batch bb are in fi / yi
    const int set = (int)(bb % NS);
    const int64_t eb = e0 + bb * STAGES;
    const int cnt = (int)min((int64_t)STAGES, e1 - eb);
    if (lane == 0) mbar_expect_tx(&bars[set], cnt * ROWB);
    if (lane < cnt) bulk_load(sm.xs + (set * STAGES + lane) * ROWF, a.feat + fi * ROWF, ROWB, &bars[set]);
    if (WITH_Y) {
#pragma unroll
      for (int i0 = 0; i0 < STAGES * S::DY; i0 += 32) {
        const int i = i0 + lane, ed = min(i / S::DY, STAGES - 1);
        const int64_t yrow = __shfl_sync(0xffffffffu, yi, ed);
        if (i < cnt * S::DY) cp_async_4(sm.ys + set * STAGES * S::DY + i, a.y + yrow * S::DY + (i - ed * S::DY));
      }
    }
    cp_async_arrive(&bars[set]);
  }
  __device__ void prologue() {
    if (warp != 0) return;
    for (int64_t bb = 0; bb < NS - 1 && bb < nb; ++bb) {
      load_idx(bb);
      issue(bb);
    }
    if (NS - 1 < nb) load_idx(NS - 1);
  }
  // start of iteration b (every warp has left batch b - 1, whose set is refilled now); returns false on a timeout
  __device__ bool begin(int64_t b) {
    if (warp == 0) {
      const int64_t bb = b + NS - 1;
      if (bb < nb) issue(bb);
      if (bb + 1 < nb) load_idx(bb + 1);
    }
    return mbar_wait(&bars[b % NS], (uint32_t)((b / NS) & 1));
  }
  // after a timeout: give copies that may still be in flight a bounded chance to land before the CTA retires
  __device__ void drain(int64_t b) {
    asm volatile("cp.async.wait_all;" ::: "memory");
    for (int64_t bb = b; bb < nb && bb < b + NS - 1; ++bb) mbar_wait(&bars[bb % NS], (uint32_t)((bb / NS) & 1));
  }
};

// ---- spec kernel: gather + outer product + per-node CG + segment sum ---------------------------------
// Warp (cq, role): channels [32 cq, 32 cq + 32), one per lane; role selects the half of the (m_y, m_feat)
// cells whose accumulators Q[cell] = sum_e y_e[m_y] x_e[m_feat] the warp keeps in registers.  When the
// last edge of a node has been added the warp turns its Q into its share of the rows,
// S[d, r] = sum_t scale[t] Q[cell(t)], stores them and clears Q.
template <class S, int CQ>
__global__ void __launch_bounds__(64 * CQ, 4 / CQ) tp_segsum_spec_kernel(FusedArgs a) {
  using SM = Smem<S, CQ>;
  constexpr int C = SM::C, ROWF = SM::ROWF, NT = 64 * CQ, NS = SM::NS;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ uint64_t bars[NS];
  SM sm(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int role = warp & 1, ch = (warp >> 1) * 32 + lane;
  const float4* sc = reinterpret_cast<const float4*>(sm.ssc + (role ? S::OT1 : 0));

  for (int t = tid; t < S::OT2; t += NT) sm.ssc[t] = __ldg(a.scale_o + t);
  if (tid == 0) {
    for (int i = 0; i < NS; ++i) mbar_init(&bars[i], 1 + 32);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  cta_sync();

  const int64_t d0 = (int64_t)blockIdx.x * a.nodes_per_cta;
  const int64_t d1 = min(d0 + a.nodes_per_cta, a.n_out);
  const int64_t e0 = a.ptr ? __ldg(a.ptr + d0) : d0;
  const int64_t e1 = a.ptr ? __ldg(a.ptr + d1) : d1;
  EdgeRing<S, CQ, true> ring(a, sm, bars, e0, e1, warp, lane);
  ring.prologue();

  float q[S::MAXCELL];
#pragma unroll
  for (int i = 0; i < S::MAXCELL; ++i) q[i] = 0.f;

  int64_t d_cur = d0;
  int64_t boundary = a.ptr ? __ldg(a.ptr + d_cur + 1) : d_cur + 1;
  auto flush = [&]() {   // a node without edges flushes a zero Q, i.e. zero rows
    float* o = a.out + d_cur * S::R * C + ch;
    if (role == 0) S::template node_r0<C>(q, sc, o);
    else S::template node_r1<C>(q, sc, o);
#pragma unroll
    for (int i = 0; i < S::MAXCELL; ++i) q[i] = 0.f;
    ++d_cur;
    if (d_cur < d1) boundary = a.ptr ? __ldg(a.ptr + d_cur + 1) : d_cur + 1;
  };

  for (int64_t b = 0; b < ring.nb; ++b) {
    if (!ring.begin(b)) {
      if (tid == 0) atomicExch(a.status, 1);
      ring.drain(b);
      return;
    }
    const int set = (int)(b % NS);
    const int64_t eb = e0 + b * STAGES;
    const int cnt = (int)min((int64_t)STAGES, e1 - eb);
    for (int s = 0; s < cnt; ++s) {
      const int64_t e = eb + s;
      while (e >= boundary) flush();
      float x[S::DF], yv[S::DY];
      const float* xr = sm.xs + (set * STAGES + s) * ROWF + ch;
      const float* yr = sm.ys + (set * STAGES + s) * S::DY;
#pragma unroll
      for (int m = 0; m < S::DF; ++m) x[m] = xr[m * C];
#pragma unroll
      for (int k = 0; k < S::DY; ++k) yv[k] = yr[k];
      if (role == 0) S::outer_r0(q, x, yv);
      else S::outer_r1(q, x, yv);
    }
    cta_sync();   // everybody is done with this set before it is refilled
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
// gy_e[k] = sum_{cells (k, m)} sum_c x_e[m, c] H_d[cell, c]  with  H_d[cell] = sum_{t in cell} scale[t] G_d[row(t)]
// built once per node in registers (same warp roles as above), then one dense dot product per edge.
template <class S, int CQ>
__global__ void __launch_bounds__(64 * CQ, 4 / CQ) tp_inner_spec_kernel(FusedArgs a) {
  using SM = Smem<S, CQ>;
  constexpr int C = SM::C, ROWF = SM::ROWF, NT = 64 * CQ, NWARP = SM::NWARP, NS = SM::NS;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ uint64_t bars[NS];
  SM sm(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int role = warp & 1, ch = (warp >> 1) * 32 + lane;
  const float4* sc = reinterpret_cast<const float4*>(sm.ssc + (role ? S::OT1 : 0));
  for (int t = tid; t < S::OT2; t += NT) sm.ssc[t] = __ldg(a.scale_o + t);
  if (tid == 0) {
    for (int i = 0; i < NS; ++i) mbar_init(&bars[i], 1 + 32);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  cta_sync();

  const int64_t d0 = (int64_t)blockIdx.x * a.nodes_per_cta;
  const int64_t d1 = min(d0 + a.nodes_per_cta, a.n_out);
  const int64_t e0 = __ldg(a.ptr + d0), e1 = __ldg(a.ptr + d1);
  EdgeRing<S, CQ, false> ring(a, sm, bars, e0, e1, warp, lane);
  ring.prologue();

  float h[S::MAXCELL];
#pragma unroll
  for (int i = 0; i < S::MAXCELL; ++i) h[i] = 0.f;
  int64_t d_cur = d0 - 1;
  int64_t boundary = e0;   // forces H to be built for the first node that has an edge
  auto next_node = [&]() {
    ++d_cur;
    boundary = __ldg(a.ptr + d_cur + 1);
    if (boundary > __ldg(a.ptr + d_cur)) {
      const float* gp = a.g + d_cur * S::R * C + ch;
      if (role == 0) S::template hbuild_r0<C>(h, sc, gp);
      else S::template hbuild_r1<C>(h, sc, gp);
    }
  };

  for (int64_t b = 0; b < ring.nb; ++b) {
    if (!ring.begin(b)) {
      if (tid == 0) atomicExch(a.status, 1);
      ring.drain(b);
      return;
    }
    const int set = (int)(b % NS), rset = (int)(b & 1);
    const int64_t eb = e0 + b * STAGES;
    const int cnt = (int)min((int64_t)STAGES, e1 - eb);
    for (int s = 0; s < cnt; ++s) {
      const int64_t e = eb + s;
      while (e >= boundary) next_node();
      float x[S::DF];
      const float* xr = sm.xs + (set * STAGES + s) * ROWF + ch;
#pragma unroll
      for (int m = 0; m < S::DF; ++m) x[m] = xr[m * C];
      float ay[S::DY];
#pragma unroll
      for (int k = 0; k < S::DY; ++k) ay[k] = 0.f;
      if (role == 0) S::dot_r0(ay, x, h);
      else S::dot_r1(ay, x, h);
      float* rd = sm.red + ((rset * STAGES + s) * NWARP + warp) * S::DY;
      warp_reduce_to_smem<S::DY>(ay, rd, lane);
    }
    cta_sync();
    // combine the warps' partial sums of this batch; the other set of partial sums is free until the next sync
    for (int i = tid; i < cnt * S::DY; i += NT) {
      const int s = i / S::DY, k = i % S::DY;
      const float* rd = sm.red + ((rset * STAGES + s) * NWARP) * S::DY + k;
      float v = rd[0];
#pragma unroll
      for (int w = 1; w < NWARP; ++w) v += rd[w * S::DY];
      const int64_t e = eb + s;
      a.out[(a.yidx ? __ldg(a.yidx + e) : e) * S::DY + k] = v;
    }
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
template <class S, int CQ>
int launch_spec(bool inner, const FusedArgs& a, cudaStream_t s) {
  constexpr size_t bytes = Smem<S, CQ>::bytes();
  auto kern = inner ? tp_inner_spec_kernel<S, CQ> : tp_segsum_spec_kernel<S, CQ>;
  static bool configured[2] = {false, false};
  if (!configured[inner]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return fail(EQT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured[inner] = true;
  }
  const unsigned grid = (unsigned)ceil_div(a.n_out, a.nodes_per_cta);
  kern<<<grid, 64 * CQ, bytes, s>>>(a);
  return check_launch(inner ? "tp_inner_spec_kernel" : "tp_segsum_spec_kernel");
}

template <class S>
bool try_spec(uint64_t key, bool inner, const FusedArgs& a, cudaStream_t s, int& rc) {
  if (key != S::KEY || a.T != S::T || a.R != S::R || a.DF != S::DF || a.DY != S::DY) return false;
  if (a.C == 128) { rc = launch_spec<S, 4>(inner, a, s); return true; }
  if (a.C == 64) { rc = launch_spec<S, 2>(inner, a, s); return true; }
  if (a.C == 32) { rc = launch_spec<S, 1>(inner, a, s); return true; }
  return false;
}

int run(bool inner, const eqt_tp_table* tab, FusedArgs a, cudaStream_t s) {
  if (a.n_out == 0 || (inner && a.n_edges == 0)) return EQT_OK;
  if ((reinterpret_cast<uintptr_t>(a.feat) & 15u) == 0 && a.status && a.scale_o && (!inner || a.ptr)) {
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
  a.scale_o = tab->scale_o;
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
