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
#include <cstdlib>

#include "tc_common.cuh"

namespace eqt {
namespace specs {
// N columns (1, 2, 4, 8 or 16) of this thread's TMEM lane, requested without waiting: several requests are followed by
// one tmem_wait_ld(), and tmem_touch() on every array keeps its uses behind the wait
template <int N> __device__ __forceinline__ void tmem_ld_nowait(uint32_t taddr, uint32_t (&r)[N]);
template <> __device__ __forceinline__ void tmem_ld_nowait<1>(uint32_t taddr, uint32_t (&r)[1]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r[0]) : "r"(taddr) : "memory");
}
template <> __device__ __forceinline__ void tmem_ld_nowait<2>(uint32_t taddr, uint32_t (&r)[2]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(taddr) : "memory");
}
template <> __device__ __forceinline__ void tmem_ld_nowait<4>(uint32_t taddr, uint32_t (&r)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
}
template <> __device__ __forceinline__ void tmem_ld_nowait<8>(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr) : "memory");
}
template <> __device__ __forceinline__ void tmem_ld_nowait<16>(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
template <int N> __device__ __forceinline__ void tmem_touch(uint32_t (&r)[N]) {
#pragma unroll
  for (int i = 0; i < N; ++i) asm volatile("" : "+r"(r[i]) :: "memory");
}
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


// ---- tensor-core segment sum -----------------------------------------------------------------------------------
// S[d, r, c] = sum_t scale[t] Q_d[m_y(t), m_feat(t), c]  with  Q_d = sum_{e -> d} y_e (x) x_e  as above, but the outer
// product - 234 of every 240 multiply-adds of the step - runs on tcgen05: per node it is the GEMM
//
//     Q_d[f, m_y] = sum_e X[e, f] Y[e, m_y],      f = (m_feat, channel): 1024 features = 8 tiles of M = 128, N = 16,
//
// whose reduction index is the edge.  Edges are taken eight at a time (one MMA k-step; the last group of a node is
// padded with zero rows), float32 operands are split into TF32 big / small parts (three MMAs per tile and group),
// and the eight accumulators of a node (128 columns) are double buffered in tensor memory.
//
// One persistent CTA per SM, 16 warps:
//   warps 0, 15   producers: bulk copies of the gathered feature rows of a group (8 x 4 KB, four requests each) into a
//                 4-slot ring, the harmonics rows by 16-byte cp.async (warp 0)
//   warps 1, 14   TMEM allocation (warp 1), MMA issue (12 of the 24 MMAs of a group each), tcgen05.commit towards
//                 splitters and contraction
//   warps 2-5,    two splitter groups taking alternate edge groups: a thread owns one TMEM lane = one (component,
//   warps 6-9     channel) of every tile, reads its eight edges' values from the ring, splits them and stores big /
//                 small into the group's A slot in tensor memory (the MMAs read A from TMEM, so the features cross
//                 shared memory once); one thread per harmonics value writes the two small B tiles
//   warps 10-13   contraction: tcgen05.ld of the finished accumulator, the 353-entry CG contraction in registers
//                 (unrolled at build time, every row produced by one lane), coalesced stores of S
// All waits are bounded; on expiry the abort flag is raised, every role leaves its loop, TMEM is freed and the
// status word is set.
namespace segtc {

constexpr int THREADS = 16 * 32;
constexpr int GE = 8;                  // edges per group (one tf32 MMA k-step)
constexpr int NS = 4;                  // ring slots
constexpr int ROWF = 1024;             // floats per gathered row (16 components x 64 channels)
constexpr int NODES_PER_CHUNK = 16;
constexpr uint32_t TMEM_COLS = 512;    // 2 x 128 accumulators + 2 x 128 A slots
constexpr uint32_t COL_A = 256;

struct Shared {
  uint64_t full[NS], empty[NS], a_ready[2], a_free[2], q_full[2], q_free[2];
  uint32_t tmem_slot;
  int abort_flag;
};

// layout of dynamic shared memory (1024-byte aligned): ring of raw rows, raw harmonics per slot, B tiles per A slot, scales
constexpr size_t XS_BYTES = (size_t)NS * GE * ROWF * 4;            // 128 KB
constexpr size_t YS_BYTES = (size_t)NS * GE * 16 * 4;              // 2 KB
constexpr size_t YB_BYTES = 2 * 2 * 2048;                          // [A slot][big, small] 16 rows x 128 B
constexpr size_t OFF_YS = XS_BYTES, OFF_YB = OFF_YS + YS_BYTES, OFF_SC = OFF_YB + YB_BYTES;

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
      : "memory");
}

// The node walk every role performs: nodes come in chunks of NODES_PER_CHUNK dealt round-robin to the CTAs.  The
// segment pointers are read two nodes ahead of their use, so the walk does not wait for a load per node.
struct Walk {
  const int64_t* ptr;
  int n_out;            // 32-bit state: the launcher checks that nodes and edges fit
  int chunk;            // current chunk
  int d_in;             // next node inside the chunk
  int p0, p1, p2;       // ptr[d], ptr[d + 1], ptr[d + 2] of the next node d
  __device__ int at(int i) const { return (int)__ldg(ptr + min(i, n_out)); }
  __device__ void prime() {
    const int d = chunk * NODES_PER_CHUNK;
    p0 = at(d); p1 = at(d + 1); p2 = at(d + 2);
  }
  __device__ Walk(const FusedArgs& a) : ptr(a.ptr), n_out((int)a.n_out), chunk(blockIdx.x), d_in(0) { prime(); }
  // next node of this CTA: returns false at the end; d = node, e0 = its first edge, deg = its edge count
  __device__ bool next(int& d, int& e0, int& deg) {
    d = chunk * NODES_PER_CHUNK + d_in;
    if (d_in >= NODES_PER_CHUNK || d >= n_out) {
      chunk += gridDim.x;
      d_in = 0;
      d = chunk * NODES_PER_CHUNK;
      if (d >= n_out) return false;
      prime();
    }
    ++d_in;
    e0 = p0;
    deg = p1 - p0;
    p0 = p1; p1 = p2; p2 = at(d + 3);
    return true;
  }
};

}  // namespace segtc

template <class S>
__global__ void __launch_bounds__(segtc::THREADS, 1) tp_segsum_tc_kernel(FusedArgs a) {
  using namespace segtc;
  using namespace tc;
  constexpr int C = 64;
  extern __shared__ unsigned char smem_raw[];
  __shared__ Shared sh;
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* xs = reinterpret_cast<float*>(base);
  float* ys = reinterpret_cast<float*>(base + OFF_YS);
  unsigned char* yb = base + OFF_YB;
  float* ssc = reinterpret_cast<float*>(base + OFF_SC);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  for (int t = tid; t < S::T; t += THREADS) ssc[t] = __ldg(a.scale + t);
  if (tid == 0) {
    sh.abort_flag = 0;
    for (int i = 0; i < NS; ++i) {
      bar_init(&sh.full[i], 1 + 32);       // expect_tx arrival + one cp.async arrival per producer lane
      bar_init(&sh.empty[i], 4);
    }
    for (int i = 0; i < 2; ++i) {
      bar_init(&sh.a_ready[i], 4);
      bar_init(&sh.a_free[i], 2);          // one commit per MMA issuer
      bar_init(&sh.q_full[i], 2);
      bar_init(&sh.q_free[i], 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&sh.tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh.tmem_slot;
  volatile int* ab = &sh.abort_flag;

  if (warp == 0 || warp == 15) {
    // ---------------- producers: warp 0 requests rows 0-3 of every group, the harmonics and arms the barrier; warp 15
    // requests rows 4-7 (the issue of a bulk copy costs a few hundred cycles per request, so two warps share it) ----
    const int row0 = warp == 0 ? 0 : GE / 2;
    Walk w(a);
    int d, e0, deg;
    int g = 0;                                       // edge groups issued
    // gather indices, one edge per lane, requested one group ahead: within a chunk the edges of consecutive nodes are
    // consecutive, so the next group starts where this one ends (row numbers fit 32 bits: checked by the launcher)
    int pf_e = -1, pf_f = 0, pf_y = 0;
    auto fetch = [&](int first, int& f, int& y) {
      const int e = first + lane;
      const bool in = lane < GE && e < (int)a.n_edges;
      f = in ? (a.fidx ? (int)__ldg(a.fidx + e) : e) : 0;
      y = in ? (a.yidx ? (int)__ldg(a.yidx + e) : e) : 0;
    };
    while (!*ab && w.next(d, e0, deg)) {
      for (int k0 = 0; k0 < deg; k0 += GE, ++g) {
        const int cnt = min(GE, deg - k0), slot = g % NS;
        const int eg = e0 + k0;
        int fi, yi;
        if (pf_e == eg) { fi = pf_f; yi = pf_y; }
        else fetch(eg, fi, yi);
        pf_e = eg + cnt;
        fetch(pf_e, pf_f, pf_y);
        if (g >= NS) {
          int ok = lane == 0 ? (int)bar_wait(&sh.empty[slot], (uint32_t)(((g / NS) - 1) & 1), ab) : 1;
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
        }
        if (warp == 0 && lane == 0) bar_expect_tx(&sh.full[slot], (uint32_t)cnt * ROWF * 4);
        __syncwarp();
        if (lane >= row0 && lane < row0 + GE / 2 && lane < cnt)
          bulk_load(xs + (size_t)(slot * GE + lane) * ROWF, a.feat + (int64_t)fi * ROWF, ROWF * 4, &sh.full[slot]);
        if (warp == 0) {
          // harmonics: lane = (edge, 16-byte chunk)
          const int ed = lane >> 2, ch = lane & 3;
          const int64_t yrow = __shfl_sync(0xffffffffu, yi, ed);
          if (ed < cnt)
            asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_addr(ys + (slot * GE + ed) * 16 + ch * 4)),
                         "l"(a.y + yrow * 16 + ch * 4) : "memory");
          cp_async_arrive(&sh.full[slot]);
        }
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (warp == 1 || warp == 14) {
    // ---------------- MMA issuers: warp 1 takes tiles 0-3, warp 14 tiles 4-7 (issue of 24 small MMAs per group from
    // one thread was the longest serial chain of the kernel) ----------------
    const int tile0 = warp == 1 ? 0 : 4;
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_tf32(16);
      Walk w(a);
      int d, e0, deg, g = 0, nq = 0;
      bool ok = true;
      while (ok && !*ab && w.next(d, e0, deg)) {
        if (deg == 0) continue;
        const int qb = nq & 1;
        if (nq >= 2 && !bar_wait(&sh.q_free[qb], (uint32_t)(((nq >> 1) - 1) & 1), ab)) break;
        tc_fence_after();
        const uint32_t dq = tmem + (uint32_t)(qb * 128);
        for (int k0 = 0; k0 < deg; k0 += GE, ++g) {
          const int G = g & 1;
          if (!bar_wait(&sh.a_ready[G], (uint32_t)((g >> 1) & 1), ab)) { ok = false; break; }
          tc_fence_after();
          const uint64_t bb = umma_desc(s32(yb + G * 4096)), bs = umma_desc(s32(yb + G * 4096 + 2048));
          const uint32_t ta = tmem + COL_A + (uint32_t)(G * 128);
          // MMAs into one accumulator execute one after the other, so the three products of a tile are issued four
          // tiles apart instead of back to back
#pragma unroll
          for (int j = 0; j < 4; ++j) umma_tf32_ta(dq + (tile0 + j) * 16, ta + (tile0 + j) * 16, bb, idesc, k0 != 0);
#pragma unroll
          for (int j = 0; j < 4; ++j) umma_tf32_ta(dq + (tile0 + j) * 16, ta + (tile0 + j) * 16, bs, idesc, 1);
#pragma unroll
          for (int j = 0; j < 4; ++j) umma_tf32_ta(dq + (tile0 + j) * 16, ta + (tile0 + j) * 16 + 8, bb, idesc, 1);
          umma_commit(&sh.a_free[G]);               // the A slot and its B tiles may be rewritten once these MMAs are done
        }
        if (!ok) break;
        umma_commit(&sh.q_full[qb]);
        ++nq;
      }
    }
  } else if (warp < 10) {
    // ---------------- splitters ----------------
    const int G = (warp - 2) >> 2, quarter = warp & 3;      // warps 2-5: group 0, 6-9: group 1; TMEM lanes 32 * (warp % 4)
    const int L = quarter * 32 + lane, h = L >> 6, c = L & 63;
    const int t128 = ((warp - 2) & 3) * 32 + lane;           // thread index inside the group: one harmonics value each
    int fo[8];                                               // offset of this lane's feature inside a row, per tile
#pragma unroll
    for (int i = 0; i < 8; ++i) fo[i] = S::tc_mfeat(h, i) * C + c;
    Walk w(a);
    int d, e0, deg, g = 0;
    bool ok = true;
    while (ok && !*ab && w.next(d, e0, deg)) {
      for (int k0 = 0; k0 < deg; k0 += GE, ++g) {
        if ((g & 1) != G) continue;
        const int cnt = min(GE, deg - k0), slot = g % NS, u = g >> 1;
        if (!bar_wait(&sh.full[slot], (uint32_t)((g / NS) & 1), ab)) { ok = false; break; }
        if (u >= 1 && !bar_wait(&sh.a_free[G], (uint32_t)((u - 1) & 1), ab)) { ok = false; break; }
        tc_fence_after();
        const float* xr = xs + (size_t)slot * GE * ROWF;
        const uint32_t ta = tmem + ((uint32_t)(quarter * 32) << 16) + COL_A + (uint32_t)(G * 128);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float v[16];
#pragma unroll
          for (int e = 0; e < GE; ++e) {
            const float x = e < cnt ? xr[e * ROWF + fo[i]] : 0.f;
            const float hi = rn_tf32(x);
            v[e] = hi;
            v[8 + e] = x - hi;
          }
          tmem_st16(ta + i * 16, v);
        }
        {   // harmonics value (edge, component) -> the two B tiles (128-byte rows, 16-byte chunks swizzled by the row)
          const int ed = t128 >> 4, m = t128 & 15;
          const float yv = ed < cnt ? ys[(slot * GE + ed) * 16 + m] : 0.f;
          const float hi = rn_tf32(yv);
          const uint32_t off = m * 128 + ((((uint32_t)ed >> 2) ^ (m & 7)) << 4) + (ed & 3) * 4;
          *reinterpret_cast<float*>(yb + G * 4096 + off) = hi;
          *reinterpret_cast<float*>(yb + G * 4096 + 2048 + off) = yv - hi;
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // B tiles: generic writes -> visible to the MMA
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          bar_arrive(&sh.a_ready[G]);
          bar_arrive(&sh.empty[slot]);
        }
      }
    }
  } else {
    // ---------------- contraction ----------------
    const int quarter = warp & 3;                            // warps 10-13 -> 2, 3, 0, 1: every quarter once
    const int L = quarter * 32 + lane, h = L >> 6, c = L & 63;
    Walk w(a);
    int d, e0, deg, nq = 0;
    while (!*ab && w.next(d, e0, deg)) {
      float* o = a.out + (int64_t)d * (S::R * C) + c;
      if (deg == 0) {                                        // node without edges: zero rows (each lane half its rows)
        for (int r = h; r < S::R; r += 2) o[r * C] = 0.f;
        continue;
      }
      const int qb = nq & 1;
      if (!bar_wait(&sh.q_full[qb], (uint32_t)((nq >> 1) & 1), ab)) break;
      tc_fence_after();
      const uint32_t tq = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(qb * 128);
      if (h == 0) S::template tc_node_h0<C>(tq, ssc, o);
      else S::template tc_node_h1<C>(tq, ssc, o);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) bar_arrive(&sh.q_free[qb]);
      ++nq;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
  if (sh.abort_flag) {
    if (tid == 0) atomicExch(a.status, 1);
    // copies that may still be in flight get a bounded chance to land before shared memory is released
    if (tid == 0)
      for (int i = 0; i < NS; ++i)
        for (int ph = 0; ph < 2; ++ph)
          for (int k = 0; k < 1024 && !bar_try(&sh.full[i], ph); ++k) __nanosleep(256);
  }
}

template <class S>
int launch_segsum_tc(const FusedArgs& a, cudaStream_t s) {
  if constexpr (S::HAS_TC) {
    constexpr size_t bytes = segtc::OFF_SC + sizeof(float) * ((S::T + 3) & ~3) + 1024;
    auto kern = tp_segsum_tc_kernel<S>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return fail(EQT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    const int64_t chunks = ceil_div(a.n_out, segtc::NODES_PER_CHUNK);
    kern<<<(unsigned)std::min<int64_t>(chunks, sm_count()), segtc::THREADS, bytes, s>>>(a);
    return check_launch("tp_segsum_tc_kernel");
  } else {
    return -1;
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

// the tensor-core kernel pays when nodes have several edges each (groups of eight) and everything is 16-byte aligned
inline bool segsum_tc_wanted(const FusedArgs& a) {
  return a.ptr && a.C == 64 && a.n_edges >= 4 * a.n_out && a.n_out < 0x7fffffffll && (reinterpret_cast<uintptr_t>(a.y) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(a.out) & 15u) == 0;
}

template <class S>
bool try_spec(uint64_t key, bool inner, const FusedArgs& a, cudaStream_t s, int& rc) {
  if (key != S::KEY || a.T != S::T || a.R != S::R || a.DF != S::DF || a.DY != S::DY) return false;
  if (!inner && S::HAS_TC && segsum_tc_wanted(a)) {
    rc = launch_segsum_tc<S>(a, s);
    if (rc >= 0) return true;
  }
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
