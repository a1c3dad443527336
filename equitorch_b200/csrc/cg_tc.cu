// Gather + Clebsch-Gordan contraction + sum over the edges of a node on tcgen05 tensor cores.
//
// For one edge the CG step is a small matrix product  inter (R x C) = B_e (R x D) * X_e (D x C):
// X_e is the gathered feature row of the edge (D components, C channels) and B_e[r, m] =
// sum_{t: row(t) = r, m_feat(t) = m} scale[t] * y_e[m_y(t)] collects the CG coefficients times the
// edge's spherical harmonics (311 non-zeros of 99 x 16 for l_max = 3).  Summing over the edges of a
// node concatenates these products along K:
//
//     S[d] (R x C) = [B_e1 | B_e2 | ...] (R x 16 deg) * [X_e1; X_e2; ...] (16 deg x C)
//
// which is run as one tcgen05 GEMM per node with M = 128 (R <= 128 rows, the rest stays zero), N = C
// and K advancing by 16 per edge, accumulator in TMEM.  The dense product does 4.5x the flops of the
// sparse CUDA-core loop, but on the tensor pipe instead of 1300 issue slots per edge.
//
//  * A operand (coefficients): built per pair of edges by the "builder" warps straight into a
//    K-major, 128B-swizzled shared-memory tile (128 rows x 32 floats).  Only the non-zero slots are
//    rewritten; the zeros were written once when the kernel started.
//  * B operand (features): TMA boxes of (32 channels, D components, 1 node) gathered by edge source
//    into the MN-major "128B swizzle, 32-byte atom" layout.
//  * float32 accuracy by the 3xTF32 split of both operands (big*big + big*small + small*big).
//  * Roles: warp 0 producer (indices, harmonics by cp.async, features by TMA), warp 1 MMA issue + TMEM, warps 2-9 builders (coefficients, split of
//    the features), warps 10-13 epilogue (one accumulator per node, double buffered, rows < R stored).
//  * All waits are bounded; on expiry the status flag is raised and the kernel winds down.
//
// Works for any table with R <= 128, D <= 16, C in {32, 64, 96, 128}; the index structure is run-time
// data (no build-time specialisation needed).
#include <algorithm>

#include "tc_common.cuh"

namespace eqt {
namespace {
using namespace tc;

constexpr int KE = 16;            // K per edge (feature components, zero padded)
constexpr int EPB = 2;            // edges per k-block (32 floats of K = one swizzle row)
constexpr int CG_BUILDER_WARPS = 8;
constexpr int CG_THREADS = (2 + CG_BUILDER_WARPS + 4) * 32;   // producer, MMA, builders, epilogue
constexpr int CG_U_PER_THREAD = 2;                            // merged table entries per builder thread
constexpr int CG_MAX_U = CG_BUILDER_WARPS * 32 * CG_U_PER_THREAD;

struct CgArgs {
  const int64_t* fidx;      // (E) feature row per edge or NULL
  const float* y;           // (Ey, DY)
  const int64_t* yidx;      // (E) or NULL
  const int64_t* ptr;       // (N + 1)
  const uint8_t* u_row;     // (U) intermediate row of each merged entry
  const uint8_t* u_m;       // (U) feature component
  const float* u_scale;     // (U, 2) scales of the (at most two) table entries merged into it
  const uint8_t* u_my;      // (U, 2) their harmonics components
  float* out;               // (N, R, C)
  int64_t n_out;
  int U, R, DF, DY, C;
  int nodes_per_chunk;
  int stages;
  int tmem_cols;
  int* status;
};

__device__ __forceinline__ void cp_async_4(void* dst_smem, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s32(dst_smem)), "l"(src) : "memory");
}
// the barrier gets one arrival (already counted in its init count) once this thread's earlier cp.async have landed
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(s32(bar)) : "memory");
}

// byte offset of element (row r, k) inside a K-major 128B-swizzled tile of 128-byte rows
__device__ __forceinline__ uint32_t a_tile_offset(int r, int k) {
  return (uint32_t)(r * 128 + ((((k >> 2) ^ (r & 7)) & 7) << 4) + ((k & 3) << 2));
}

__global__ void __launch_bounds__(CG_THREADS, 1)
cg_segsum_tc_kernel(const __grid_constant__ CUtensorMap map_x, CgArgs p) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ uint64_t bar_full[8], bar_ready[8], bar_empty[8], bar_acc_full[2], bar_acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ __align__(16) float ys[8][EPB * KE];   // harmonics rows of the k-block in each stage
  __shared__ int4 kb_meta[8];                        // {edges in the k-block, first of its node, last of its node, stop}

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int atoms = p.C / 32;
  const uint32_t a_bytes = TILE_M * 128;                       // one coefficient tile (big or small)
  const uint32_t xbox = KE * 128;                              // one (edge, channel atom) box: 16 rows x 128 B
  const uint32_t x_bytes = EPB * atoms * xbox;                 // features of a k-block (big or small)
  const uint32_t stage_bytes = 2 * a_bytes + 2 * x_bytes;      // [A big][A small][X big][X small]
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // zero every stage once: coefficient slots that are never written stay zero, feature rows >= DF too
  for (uint32_t i = tid; i < (uint32_t)p.stages * stage_bytes / 16; i += CG_THREADS)
    reinterpret_cast<uint4*>(base)[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < p.stages; ++s) {
      bar_init(&bar_full[s], 1 + 32);           // lane 0's expect_tx + one cp.async arrival per producer lane
      bar_init(&bar_ready[s], CG_BUILDER_WARPS);
      bar_init(&bar_empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      bar_init(&bar_acc_full[a], 1);
      bar_init(&bar_acc_empty[a], 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&tmem_slot)), "r"(p.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the zero fill must be visible to TMA / MMA
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  volatile int* ab = &abort_flag;
  const int64_t chunks = ceil_div(p.n_out, p.nodes_per_chunk);

#include "cg_tc_roles.inc"

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(p.tmem_cols) : "memory");
  }
  if (tid == 0 && abort_flag) atomicExch(p.status, 4);
}

}  // namespace
}  // namespace eqt

#include "cg_tc_host.inc"
