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
//    are consumed.  A warp handles 32 or 64 channels (one or two per lane) and one quarter of the
//    cells, chosen so that every intermediate row is produced by exactly one warp from its own
//    registers.  No
//    atomics: the edges of a node are consecutive.  The adjoint runs the same scheme backwards:
//    H[cell] = sum_t scale[t] G_d[row(t)] once per node, then a dense dot product per edge.
//  * "generic": table-driven, one thread per output element; any structure, any channel count.
#include <algorithm>

#include "common.cuh"

namespace eqt {
namespace specs {
template <int CPL> __device__ __forceinline__ void ld_lane(float (&x)[CPL], const float* p) {
  if constexpr (CPL == 2) { const float2 v = *reinterpret_cast<const float2*>(p); x[0] = v.x; x[1] = v.y; }
  else x[0] = p[0];
}
template <int CPL> __device__ __forceinline__ void ldg_lane(float (&x)[CPL], const float* p) {
  if constexpr (CPL == 2) { const float2 v = __ldg(reinterpret_cast<const float2*>(p)); x[0] = v.x; x[1] = v.y; }
  else x[0] = __ldg(p);
}
template <int CPL> __device__ __forceinline__ void st_lane(float* p, const float (&v)[CPL]) {
  if constexpr (CPL == 2) *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
  else p[0] = v[0];
}
#define EQT_LDX(X, P) ld_lane<CPL>(X, P)
#define EQT_LDG(X, P) ldg_lane<CPL>(X, P)
#define EQT_STX(P, V) st_lane<CPL>(P, V)
#define EQT_FMA(ACC, A, S) do { _Pragma("unroll") for (int k_ = 0; k_ < CPL; ++k_) (ACC)[k_] = fmaf((A)[k_], (S), (ACC)[k_]); } while (0)
#define EQT_MUL(ACC, A, S) do { _Pragma("unroll") for (int k_ = 0; k_ < CPL; ++k_) (ACC)[k_] = (A)[k_] * (S); } while (0)
#define EQT_ZERO(V) do { _Pragma("unroll") for (int k_ = 0; k_ < CPL; ++k_) (V)[k_] = 0.f; } while (0)
#define EQT_DOT(ACC, X, H) do { _Pragma("unroll") for (int k_ = 0; k_ < CPL; ++k_) (ACC) = fmaf((X)[k_], (H)[k_], (ACC)); } while (0)
#define EQT_DOT0(ACC, X, H) do { (ACC) = (X)[0] * (H)[0]; _Pragma("unroll") for (int k_ = 1; k_ < CPL; ++k_) (ACC) = fmaf((X)[k_], (H)[k_], (ACC)); } while (0)
#include "generated/tp_specs.inc"
#undef EQT_LDX
#undef EQT_LDG
#undef EQT_STX
#undef EQT_FMA
#undef EQT_MUL
#undef EQT_ZERO
#undef EQT_DOT
#undef EQT_DOT0
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
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
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

// Shared memory of the spec kernels: a lane holds CPL channels, a CTA has CG groups of four warps (one
// warp per role), i.e. C = 32 CPL CG channels, and a ring of NS batches of STAGES edges.
template <class S, int CPL, int CG>
struct Smem {
  static constexpr int C = 32 * CPL * CG, NWARP = 4 * CG, NT = 32 * NWARP, ROWF = S::DF * C;
  static constexpr int NS = 4;
  float* xs;      // [NS][STAGES][DF * C] gathered feature rows
  float* ys;      // [NS][STAGES][DY] harmonics rows of the batch (segment sum)
  float* ssc;     // [OT4] scales in role order
  float* red;     // [2][STAGES][NWARP][DY] per-warp partial grad_y, two sets (adjoint)
  __device__ explicit Smem(unsigned char* base) {
    xs = reinterpret_cast<float*>(base);
    ys = xs + NS * STAGES * ROWF;
    ssc = ys + NS * STAGES * S::DY;
    red = ssc + S::OT4;
  }
  static constexpr size_t bytes() {
    return sizeof(float) * (NS * STAGES * ROWF + NS * STAGES * S::DY + S::OT4 + 2 * STAGES * NWARP * S::DY) + 64;
  }
};

// Ring of edge batches filled ahead of their use by warp 0: feature rows by bulk copies (lane s copies
// the row of edge s), harmonics elements by 4-byte cp.async, both completing on the batch's "full"
// mbarrier (1 arrival for the expected bytes + 1 per lane of warp 0 for its cp.async).  The gather
// indices of a batch are read one iteration before they are needed, so no global-memory latency
// sits between two batches.
//   SYNCED:  the kernel ends every batch with a CTA barrier; batch b + NS - 1 is issued at the start of
//            iteration b into the set batch b - 1 has just left.
//   !SYNCED: warps run free; each releases a batch on its "empty" mbarrier, and batch b + NS - 2 is issued
//            at the start of warp 0's iteration b once every warp has released batch b - 2.
template <class S, int CPL, int CG, bool WITH_Y, bool SYNCED>
struct EdgeRing {
  using SM = Smem<S, CPL, CG>;
  static constexpr int NS = SM::NS, ROWF = SM::ROWF, LEAD = SYNCED ? NS - 1 : NS - 2;
  static constexpr uint32_t ROWB = ROWF * sizeof(float);
  const FusedArgs& a;
  SM& sm;
  uint64_t* full;
  uint64_t* empty;
  int64_t e0;               // first edge of the CTA; everything else counts edges / batches from here in 32 bits
  int ne, nb;
  int warp, lane;
  int64_t fi = 0, yi = 0;   // warp 0, lane s: indices of edge s of the next batch to issue

  __device__ EdgeRing(const FusedArgs& a_, SM& sm_, uint64_t* full_, uint64_t* empty_, int64_t e0_, int ne_,
                      int warp_, int lane_)
      : a(a_), sm(sm_), full(full_), empty(empty_), e0(e0_), ne(ne_), nb((ne_ + STAGES - 1) / STAGES), warp(warp_),
        lane(lane_) {}

  __device__ static void init(uint64_t* full_, uint64_t* empty_) {   // one thread
    for (int i = 0; i < NS; ++i) {
      mbar_init(&full_[i], 1 + 32);
      mbar_init(&empty_[i], SM::NWARP);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __device__ void load_idx(int bb) {
    const int er = bb * STAGES + lane;
    if (lane < STAGES && er < ne) {
      const int64_t e = e0 + er;
      fi = a.fidx ? __ldg(a.fidx + e) : e;
      if (WITH_Y) yi = a.yidx ? __ldg(a.yidx + e) : e;
    }
  }
  __device__ void issue(int bb) {   // whole warp 0; indices of batch bb are in fi / yi
    const int set = bb % NS;
    const int cnt = min(STAGES, ne - bb * STAGES);
    if (lane == 0) mbar_expect_tx(&full[set], cnt * ROWB);
    if (lane < cnt) bulk_load(sm.xs + (set * STAGES + lane) * ROWF, a.feat + fi * ROWF, ROWB, &full[set]);
    if (WITH_Y) {
#pragma unroll
      for (int i0 = 0; i0 < STAGES * S::DY; i0 += 32) {
        const int i = i0 + lane, ed = min(i / S::DY, STAGES - 1);
        const int64_t yrow = __shfl_sync(0xffffffffu, yi, ed);
        if (i < cnt * S::DY) cp_async_4(sm.ys + set * STAGES * S::DY + i, a.y + yrow * S::DY + (i - ed * S::DY));
      }
    }
    cp_async_arrive(&full[set]);
  }
  __device__ void prologue() {
    if (warp != 0) return;
    for (int bb = 0; bb < LEAD && bb < nb; ++bb) {
      load_idx(bb);
      issue(bb);
    }
    if (LEAD < nb) load_idx(LEAD);
  }
  // start of iteration b; returns false on a timeout
  __device__ bool begin(int b) {
    if (warp == 0) {
      const int bb = b + LEAD;
      if (bb < nb) {
        if (!SYNCED && bb >= NS) {   // the set's previous batch must have been released by every warp
          int ok = (lane == 0) ? (int)mbar_wait(&empty[bb % NS], (uint32_t)(((bb / NS) - 1) & 1)) : 0;
          ok = __shfl_sync(0xffffffffu, ok, 0);
          __syncwarp();
          if (!ok) return false;
        }
        issue(bb);
      }
      if (bb + 1 < nb) load_idx(bb + 1);
    }
    return mbar_wait(&full[b % NS], (uint32_t)((b / NS) & 1));
  }
  __device__ void release(int b) {   // !SYNCED: this warp is done with batch b
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[b % NS]);
  }
  // after a timeout: give copies that may still be in flight a bounded chance to land before the CTA retires
  __device__ void drain(int b) {
    asm volatile("cp.async.wait_all;" ::: "memory");
    for (int bb = b; bb < nb && bb < b + LEAD; ++bb) mbar_wait(&full[bb % NS], (uint32_t)((bb / NS) & 1));
  }
};

template <class S, int CPL, int CG>
__device__ __forceinline__ const float4* role_scales(const Smem<S, CPL, CG>& sm, int role) {
  return reinterpret_cast<const float4*>(sm.ssc + (role == 0 ? S::OT0 : role == 1 ? S::OT1 : role == 2 ? S::OT2 : S::OT3));
}

// ---- spec kernel: gather + outer product + per-node CG + segment sum ---------------------------------
// Warp (cg, role): channels [32 CPL cg, 32 CPL (cg + 1)), CPL per lane; role selects the quarter of the
// (m_y, m_feat) cells whose accumulators Q[cell] = sum_e y_e[m_y] x_e[m_feat] the warp keeps in
// registers.  When the last edge of a node has been added the warp turns its Q into its share of the
// rows, S[d, r] = sum_t scale[t] Q[cell(t)], stores them and clears Q.  Warps never wait for each other.
template <class S, int CPL, int CG>
__global__ void __launch_bounds__(128 * CG, CG == 1 ? 3 : 1) tp_segsum_spec_kernel(FusedArgs a) {
  using SM = Smem<S, CPL, CG>;
  constexpr int C = SM::C, ROWF = SM::ROWF, NT = SM::NT, NS = SM::NS;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ uint64_t full[NS], empty[NS];
  SM sm(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int role = warp & 3, ch = ((warp >> 2) * 32 + lane) * CPL;
  const float4* sc = role_scales(sm, role);

  for (int t = tid; t < S::OT4; t += NT) sm.ssc[t] = __ldg(a.scale_o + t);
  using Ring = EdgeRing<S, CPL, CG, true, false>;
  if (tid == 0) Ring::init(full, empty);
  cta_sync();

  const int64_t d0 = (int64_t)blockIdx.x * a.nodes_per_cta;
  const int nd = (int)min((int64_t)a.nodes_per_cta, a.n_out - d0);
  const int64_t e0 = a.ptr ? __ldg(a.ptr + d0) : d0;
  const int ne = (int)((a.ptr ? __ldg(a.ptr + d0 + nd) : d0 + nd) - e0);
  Ring ring(a, sm, full, empty, e0, ne, warp, lane);
  ring.prologue();

  float q[S::MAXCELL][CPL];
#pragma unroll
  for (int i = 0; i < S::MAXCELL; ++i)
#pragma unroll
    for (int k = 0; k < CPL; ++k) q[i][k] = 0.f;

  // nodes and edges are counted from the CTA's first (d0, e0) in 32 bits to save registers
  const int64_t* ptr = a.ptr ? a.ptr + d0 : nullptr;
  float* o = a.out + d0 * S::R * C + ch;
  int d_cur = 0;
  int boundary = ptr ? (int)(__ldg(ptr + 1) - e0) : 1;   // first edge of the next node
  auto flush = [&]() __attribute__((always_inline)) {   // a node without edges flushes a zero Q, i.e. zero rows
    if (role == 0) S::template node_r0<CPL, C>(q, sc, o);
    else if (role == 1) S::template node_r1<CPL, C>(q, sc, o);
    else if (role == 2) S::template node_r2<CPL, C>(q, sc, o);
    else S::template node_r3<CPL, C>(q, sc, o);
#pragma unroll
    for (int i = 0; i < S::MAXCELL; ++i)
#pragma unroll
      for (int k = 0; k < CPL; ++k) q[i][k] = 0.f;
    ++d_cur;
    o += S::R * C;
    if (d_cur < nd) boundary = ptr ? (int)(__ldg(ptr + d_cur + 1) - e0) : d_cur + 1;
  };

  for (int b = 0; b < ring.nb; ++b) {
    if (!ring.begin(b)) {
      if (lane == 0) atomicExch(a.status, 1);
      ring.drain(b);
      return;
    }
    const int set = b % NS;
    const int cnt = min(STAGES, ne - b * STAGES);
    for (int s = 0; s < cnt; ++s) {
      const int e = b * STAGES + s;
      while (e >= boundary) flush();
      float yv[S::DY];
      const float* xr = sm.xs + (set * STAGES + s) * ROWF + ch;
      const float* yr = sm.ys + (set * STAGES + s) * S::DY;
      if constexpr (S::DY % 4 == 0) {
#pragma unroll
        for (int k = 0; k < S::DY; k += 4) {
          const float4 v = *reinterpret_cast<const float4*>(yr + k);
          yv[k] = v.x; yv[k + 1] = v.y; yv[k + 2] = v.z; yv[k + 3] = v.w;
        }
      } else {
#pragma unroll
        for (int k = 0; k < S::DY; ++k) yv[k] = yr[k];
      }
      if (role == 0) S::template outer_r0<CPL, C>(q, xr, yv);
      else if (role == 1) S::template outer_r1<CPL, C>(q, xr, yv);
      else if (role == 2) S::template outer_r2<CPL, C>(q, xr, yv);
      else S::template outer_r3<CPL, C>(q, xr, yv);
    }
    ring.release(b);
  }
  while (d_cur < nd) flush();
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
template <class S, int CPL, int CG>
__global__ void __launch_bounds__(128 * CG, CG == 1 ? 3 : 1) tp_inner_spec_kernel(FusedArgs a) {
  using SM = Smem<S, CPL, CG>;
  constexpr int C = SM::C, ROWF = SM::ROWF, NT = SM::NT, NWARP = SM::NWARP, NS = SM::NS;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ uint64_t full[NS], empty[NS];
  SM sm(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int role = warp & 3, ch = ((warp >> 2) * 32 + lane) * CPL;
  const float4* sc = role_scales(sm, role);
  for (int t = tid; t < S::OT4; t += NT) sm.ssc[t] = __ldg(a.scale_o + t);
  using Ring = EdgeRing<S, CPL, CG, false, true>;
  if (tid == 0) Ring::init(full, empty);
  cta_sync();

  const int64_t d0 = (int64_t)blockIdx.x * a.nodes_per_cta;
  const int nd = (int)min((int64_t)a.nodes_per_cta, a.n_out - d0);
  const int64_t* ptr = a.ptr + d0;
  const int64_t e0 = __ldg(ptr);
  const int ne = (int)(__ldg(ptr + nd) - e0);
  Ring ring(a, sm, full, empty, e0, ne, warp, lane);
  ring.prologue();

  float h[S::MAXCELL][CPL];
#pragma unroll
  for (int i = 0; i < S::MAXCELL; ++i)
#pragma unroll
    for (int k = 0; k < CPL; ++k) h[i][k] = 0.f;
  // nodes and edges are counted from the CTA's first (d0, e0) in 32 bits to save registers
  const float* gp = a.g + (d0 - 1) * S::R * C + ch;
  int d_cur = -1;
  int boundary = 0;   // forces H to be built for the first node that has an edge
  auto next_node = [&]() __attribute__((always_inline)) {
    ++d_cur;
    gp += S::R * C;
    const int begin = boundary;
    boundary = (int)(__ldg(ptr + d_cur + 1) - e0);
    if (boundary > begin) {
      if (role == 0) S::template hbuild_r0<CPL, C>(h, sc, gp);
      else if (role == 1) S::template hbuild_r1<CPL, C>(h, sc, gp);
      else if (role == 2) S::template hbuild_r2<CPL, C>(h, sc, gp);
      else S::template hbuild_r3<CPL, C>(h, sc, gp);
    }
  };

  for (int b = 0; b < ring.nb; ++b) {
    if (!ring.begin(b)) {
      if (lane == 0) atomicExch(a.status, 1);
      ring.drain(b);
      return;
    }
    const int set = b % NS, rset = b & 1;
    const int cnt = min(STAGES, ne - b * STAGES);
    for (int s = 0; s < cnt; ++s) {
      const int e = b * STAGES + s;
      while (e >= boundary) next_node();
      const float* xr = sm.xs + (set * STAGES + s) * ROWF + ch;
      float ay[S::DY];   // fully written by dot_r*
      if (role == 0) S::template dot_r0<CPL, C>(ay, xr, h);
      else if (role == 1) S::template dot_r1<CPL, C>(ay, xr, h);
      else if (role == 2) S::template dot_r2<CPL, C>(ay, xr, h);
      else S::template dot_r3<CPL, C>(ay, xr, h);
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
      const int64_t e = e0 + b * STAGES + s;
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
template <class S, int CPL, int CG>
int launch_spec(bool inner, const FusedArgs& a, cudaStream_t s) {
  constexpr size_t bytes = Smem<S, CPL, CG>::bytes();
  auto kern = inner ? tp_inner_spec_kernel<S, CPL, CG> : tp_segsum_spec_kernel<S, CPL, CG>;
  // the attribute belongs to the current device's context, so it is set on every launch (a cheap host-side call)
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) return fail(EQT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  const unsigned grid = (unsigned)ceil_div(a.n_out, a.nodes_per_cta);
  kern<<<grid, 128 * CG, bytes, s>>>(a);
  return check_launch(inner ? "tp_inner_spec_kernel" : "tp_segsum_spec_kernel");
}

template <class S>
bool try_spec(uint64_t key, bool inner, const FusedArgs& a, cudaStream_t s, int& rc) {
  if (key != S::KEY || a.T != S::T || a.R != S::R || a.DF != S::DF || a.DY != S::DY) return false;
  if (a.C == 128) { rc = launch_spec<S, 2, 2>(inner, a, s); return true; }
  if (a.C == 64) { rc = launch_spec<S, 2, 1>(inner, a, s); return true; }
  if (a.C == 32) { rc = launch_spec<S, 1, 1>(inner, a, s); return true; }
  return false;
}

int run(bool inner, const eqt_tp_table* tab, FusedArgs a, cudaStream_t s) {
  if (a.n_out == 0 || (inner && a.n_edges == 0)) return EQT_OK;
  if ((reinterpret_cast<uintptr_t>(a.feat) & 15u) == 0 && a.status && a.scale_o && (!inner || a.ptr) && a.n_edges < 0x7fffffffll) {
    // nodes per CTA: keep every SM busy with several CTAs but amortise the pipeline prologue
    int64_t per = std::max<int64_t>(1, a.n_out / ((int64_t)sm_count() * 16));
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
    tp_inner_generic_kernel<<<flat_grid(a.n_edges, 4, 16), 128, bytes, s>>>(a);
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
