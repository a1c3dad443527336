// Node-level channel mixing on the 5th-generation tensor cores (tcgen05, accumulators in TMEM).
//
// For one output irrep (a "block": `dim` components, `paths` coupling paths into it) the weight
// step of the layer is a plain GEMM
//
//     out[(node, m), co] = sum_{kk} A[(node, m), kk] * Bt[co, kk],      kk = (path, ci)
//
// because the intermediate rows of a fixed output component are contiguous in memory: row
// (node, m) of A is the slice S[node, in_row0 + m*paths : in_row0 + (m+1)*paths, :] of the
// per-node intermediate, K = paths * C_in floats long.  A is described to TMA as a 3-D tensor
// (kk, m, node) so that one box of (32 floats, dim, nodes_per_tile) lands in shared memory as up
// to 128 consecutive 128-byte rows in the 128B-swizzled K-major layout tcgen05.mma reads.
//
// Precision: float32 results are required to 1e-5, which a single TF32 product (10 mantissa
// bits) cannot give.  Each operand is split as x = big + small with big = x with the 13 low
// mantissa bits cleared (exactly representable in TF32) and small = x - big (exact), and three
// kind::tf32 MMAs accumulate big*big + big*small + small*big in float32 in TMEM; the dropped
// small*small term is below 2^-22 relative.  The weights are split once on the host side of the
// call, the activations by four "splitter" warps between the TMA arrival and the MMA issue.
//
// Roles inside a CTA of 10 warps (one persistent CTA per SM, tiles of up to 128 (node, m) rows):
//   warp 0      TMA producer (one elected lane), ring of `stages` k-blocks of 32 floats
//   warp 1      TMEM allocation, MMA issue (one elected lane), tcgen05.commit to free stages
//   warps 2-5   split A in place (big) and into a second buffer (small), fence to the async proxy
//   warps 6-9   epilogue: tcgen05.ld of the finished accumulator (double buffered in TMEM),
//               float4 stores of the valid rows
// Every wait on an mbarrier is bounded; on expiry the kernel raises the status flag, stops
// issuing work, frees its TMEM and returns.
#include <algorithm>
#include <vector>

#include "tc_common.cuh"

namespace eqt {
namespace {
using namespace tc;

constexpr int MAX_JOBS = 8;

struct alignas(64) JobDev {
  CUtensorMap map_a, map_bb, map_bs;        // A (3-D: k, m, node), B big / small (2-D: k, column)
  float* out;                               // first output element of (node 0, m 0)
  int64_t out_node_stride, out_m_stride;    // in floats; a row holds n_cols contiguous floats
  int64_t tile_begin;                       // position of the job's first tile in the launch's work list
  int dim;                                  // rows per node
  int npt;                                  // nodes per tile (npt * dim <= 128)
  int kblocks;                              // K / 32
  int n_cols;                               // N of this job
};

struct MixLaunch {
  JobDev job[MAX_JOBS];
  int64_t n;            // nodes
  int64_t total_tiles;
  int num_jobs;
  int max_cols;         // largest N among the jobs: fixes the stage layout and the TMEM split
  int stages;
  int tmem_cols;        // power of two >= 2 * max_cols (+ 64 per stage with a_in_tmem)
  int a_in_tmem;        // split A operand lives in tensor memory instead of shared memory
  int issuers;          // MMA issuer warps (2 when two accumulators per tile fit tensor memory)
  int* status;
};

}  // namespace
}  // namespace eqt

#include "mix_tc_kernel.inc"
#include "wgrad_tc_kernel.inc"
#include "vecmat_tc_kernel.inc"

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
namespace eqt {
namespace {

struct GemmJob {
  const float* a;            // first element of (node 0, m 0, k 0)
  int64_t K;                 // reduction length (multiple of 32); row (node, m) holds K contiguous floats
  int dim;                   // rows per node
  int64_t a_m_stride, a_node_stride;       // floats
  const float* b_big;        // (N, K) row-major
  const float* b_small;
  int N;                     // multiple of 16, <= 256
  float* out;
  int64_t out_node_stride, out_m_stride;   // floats
};

int launch_jobs(const GemmJob* jobs, int count, int64_t n, int* status, cudaStream_t st) {
  {   // per device / context, so set on every call (a cheap host-side call)
    cudaError_t e = cudaFuncSetAttribute(mix_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) return fail(EQT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  }
  for (int first = 0; first < count; first += MAX_JOBS) {
    const int m = std::min(MAX_JOBS, count - first);
    MixLaunch L{};
    L.n = n; L.num_jobs = m; L.status = status;
    for (int q = 0; q < m; ++q) L.max_cols = std::max(L.max_cols, jobs[first + q].N);
    const uint32_t a_bytes = TILE_M * KB * 4, b_bytes = (uint32_t)L.max_cols * KB * 4;
    uint32_t stage_bytes = 2 * a_bytes + 2 * b_bytes;
    const size_t epi_bytes = EPI_PATCH_BYTES;                  // the epilogue warps' transpose patches behind the ring
    const size_t ring_budget = 220 * 1024 - 1024 - epi_bytes;
    L.stages = (int)std::min<size_t>(8, ring_budget / stage_bytes);
    {   // A through tensor memory when at least four stages of 64 columns fit beside the two accumulators
      const uint32_t sb = a_bytes + 2 * b_bytes;
      const int st = (int)std::min<size_t>(std::min<size_t>(8, ring_budget / sb), (512 - 2 * L.max_cols) / 64);
      if (st >= 4) {
        L.a_in_tmem = 1;
        L.stages = st;
        stage_bytes = sb;
      }
    }
    L.issuers = 1;
    if (L.a_in_tmem && 4 * L.max_cols + 64 * 4 <= 512) {      // two accumulators per tile and at least four A slots
      L.issuers = 2;
      L.stages = std::min(L.stages, (512 - 4 * L.max_cols) / 64);
    }
    if (L.stages < 2) return fail(EQT_ERR_UNSUPPORTED, "tile too wide for the shared-memory ring");
    // the epilogue reads accumulators in groups of 32 columns, so the second one is padded to a multiple of 32
    const int acc_cols = (2 * L.issuers - 1) * L.max_cols + (L.max_cols + 31) / 32 * 32;
    L.tmem_cols = 32;
    while (L.tmem_cols < std::max(acc_cols, 2 * L.issuers * L.max_cols + (L.a_in_tmem ? 64 * L.stages : 0))) L.tmem_cols <<= 1;
    int64_t total = 0;
    for (int q = 0; q < m; ++q) {
      const GemmJob& j = jobs[first + q];
      JobDev& d = L.job[q];
      d.out = j.out; d.out_node_stride = j.out_node_stride; d.out_m_stride = j.out_m_stride;
      d.dim = j.dim; d.npt = TILE_M / j.dim; d.kblocks = (int)(j.K / KB); d.n_cols = j.N;
      d.tile_begin = total;
      total += ceil_div(n, d.npt);
      {
        cuuint64_t dims[3] = {(cuuint64_t)j.K, (cuuint64_t)j.dim, (cuuint64_t)n};
        cuuint64_t strides[2] = {(cuuint64_t)j.a_m_stride * 4, (cuuint64_t)j.a_node_stride * 4};
        cuuint32_t box[3] = {KB, (cuuint32_t)j.dim, (cuuint32_t)d.npt};
        if (int rc = make_map(&d.map_a, j.a, 3, dims, strides, box)) return rc;
      }
      {
        cuuint64_t dims[2] = {(cuuint64_t)j.K, (cuuint64_t)j.N};
        cuuint64_t strides[1] = {(cuuint64_t)j.K * 4};
        cuuint32_t box[2] = {KB, (cuuint32_t)j.N};
        if (int rc = make_map(&d.map_bb, j.b_big, 2, dims, strides, box)) return rc;
        if (int rc = make_map(&d.map_bs, j.b_small, 2, dims, strides, box)) return rc;
      }
    }
    L.total_tiles = total;
    const unsigned grid = (unsigned)std::min<int64_t>(total, sm_count());
    mix_tc_kernel<<<grid, TC_THREADS + 32, (size_t)L.stages * stage_bytes + 1024 + epi_bytes, st>>>(L);
    if (int rc = check_launch("mix_tc_kernel")) return rc;
  }
  return EQT_OK;
}

int check_common(const void* a, const void* b, const void* c, const void* d, const eqt_mix_block* blocks, int32_t* status,
                 int64_t n, int32_t rows, int32_t comps, int32_t cin, int32_t cout, int32_t num_blocks) {
  if (n < 0 || rows <= 0 || comps <= 0 || cin <= 0 || cout <= 0 || num_blocks < 0) return fail(EQT_ERR_BAD_ARGUMENT, "bad sizes");
  if (n == 0 || num_blocks == 0) return -1;
  if (!a || !b || !c || !d || !blocks || !status) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
       reinterpret_cast<uintptr_t>(d)) & 15u)
    return fail(EQT_ERR_UNSUPPORTED, "tensor-core mix needs 16-byte aligned operands");
  if (n > 0x7fffffffll) return fail(EQT_ERR_UNSUPPORTED, "too many nodes for one TMA coordinate");
  return EQT_OK;
}

}  // namespace
}  // namespace eqt

extern "C" int eqt_mix_tc(const float* s, const float* w_big, const float* w_small, float* out, int64_t n,
                          int32_t rows, int32_t comps, int32_t cin, int32_t cout, const eqt_mix_block* blocks,
                          int32_t num_blocks, int32_t* status, void* stream) {
  using namespace eqt;
  if (int rc = check_common(s, w_big, w_small, out, blocks, status, n, rows, comps, cin, cout, num_blocks))
    return rc < 0 ? EQT_OK : rc;
  if (cin % KB != 0 || cout % 16 != 0 || cout > 256)
    return fail(EQT_ERR_UNSUPPORTED, "tensor-core mix needs C_in %% 32 == 0 and C_out %% 16 == 0, C_out <= 256");
  std::vector<GemmJob> jobs;
  for (int b = 0; b < num_blocks; ++b) {
    const eqt_mix_block& blk = blocks[b];
    if (blk.dim <= 0 || blk.dim > TILE_M || blk.paths <= 0) return fail(EQT_ERR_BAD_ARGUMENT, "bad block %d", b);
    GemmJob j{};
    j.K = (int64_t)blk.paths * cin; j.dim = blk.dim;
    j.a = s + (int64_t)blk.in_row0 * cin; j.a_m_stride = j.K; j.a_node_stride = (int64_t)rows * cin;
    j.b_big = w_big + blk.w_offset; j.b_small = w_small + blk.w_offset; j.N = cout;
    j.out = out + (int64_t)blk.out_row0 * cout; j.out_node_stride = (int64_t)comps * cout; j.out_m_stride = cout;
    jobs.push_back(j);
  }
  return launch_jobs(jobs.data(), (int)jobs.size(), n, status, static_cast<cudaStream_t>(stream));
}

extern "C" int eqt_mix_tc_transposed(const float* g, const float* w_big, const float* w_small, float* g_inter,
                                     int64_t n, int32_t rows, int32_t comps, int32_t cin, int32_t cout,
                                     const eqt_mix_block* blocks, int32_t num_blocks, int32_t* status, void* stream) {
  using namespace eqt;
  if (int rc = check_common(g, w_big, w_small, g_inter, blocks, status, n, rows, comps, cin, cout, num_blocks))
    return rc < 0 ? EQT_OK : rc;
  if (cout % KB != 0 || cin % 16 != 0)
    return fail(EQT_ERR_UNSUPPORTED, "transposed tensor-core mix needs C_out %% 32 == 0 and C_in %% 16 == 0");
  std::vector<GemmJob> jobs;
  for (int b = 0; b < num_blocks; ++b) {
    const eqt_mix_block& blk = blocks[b];
    if (blk.dim <= 0 || blk.dim > TILE_M || blk.paths <= 0) return fail(EQT_ERR_BAD_ARGUMENT, "bad block %d", b);
    const int64_t width = (int64_t)blk.paths * cin;        // floats per (node, m) row of g_inter
    const int chunk_max = (256 / cin) > 0 ? (256 / cin) * cin : 0;
    if (chunk_max == 0) return fail(EQT_ERR_UNSUPPORTED, "C_in > 256");
    for (int64_t c0 = 0; c0 < width; c0 += chunk_max) {
      GemmJob j{};
      j.K = cout; j.dim = blk.dim;
      j.a = g + (int64_t)blk.out_row0 * cout; j.a_m_stride = cout; j.a_node_stride = (int64_t)comps * cout;
      j.b_big = w_big + blk.w_offset + c0 * cout; j.b_small = w_small + blk.w_offset + c0 * cout;
      j.N = (int)std::min<int64_t>(chunk_max, width - c0);
      j.out = g_inter + (int64_t)blk.in_row0 * cin + c0; j.out_node_stride = (int64_t)rows * cin; j.out_m_stride = width;
      jobs.push_back(j);
    }
  }
  return launch_jobs(jobs.data(), (int)jobs.size(), n, status, static_cast<cudaStream_t>(stream));
}

namespace eqt {
namespace {

// Launch of the weight-gradient kernel instance for the batch's output columns: one CTA per (block, split, M slice).
int launch_wgrad(const WgradBatch& b, size_t smem, cudaStream_t st) {
  cudaError_t e = b.n_cols <= 64
                      ? cudaFuncSetAttribute(wgrad_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)
                      : cudaFuncSetAttribute(wgrad_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
  if (e != cudaSuccess) return fail(EQT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  const WgradBlock& last = b.blk[b.count - 1];
  const unsigned grid = (unsigned)(last.cta_begin + last.splits * last.m_tiles);
  if (b.n_cols <= 64)
    wgrad_tc_kernel<64><<<grid, WgradCfg<64>::THREADS, smem, st>>>(b);
  else
    wgrad_tc_kernel<128><<<grid, WgradCfg<128>::THREADS, smem, st>>>(b);
  return check_launch("wgrad_tc_kernel");
}

// Launch shape of the weight-gradient GEMM of one block: reduction rows per tile, M tiles, node splits and the
// floats of scratch the per-CTA partial sums need.  Returns an error code for blocks that do not fit.
struct WgradShape { int npt, rows_pad, m_tiles, splits, stages, chunk_tiles; size_t stage_bytes; int64_t K, need; };
int wgrad_shape(const eqt_mix_block& blk, int b, int64_t n, int cin, int cout, WgradShape* w) {
  if (blk.dim <= 0 || blk.dim > TILE_M || blk.paths <= 0) return fail(EQT_ERR_BAD_ARGUMENT, "bad block %d", b);
  const int b_boxes = cout / 32;
  const size_t budget = 220 * 1024 - 1024;
  w->K = (int64_t)blk.paths * cin;                               // M extent of this GEMM
  w->m_tiles = (int)ceil_div(w->K, 128);
  // Reduction rows per tile: the most that leaves three stages in shared memory (with two, the TMA, split and MMA
  // phases of the ring cannot overlap; smaller tiles pay more per-box issue cost per byte); whole nodes, padded with
  // zero rows to a multiple of 8.
  const size_t bytes_per_row = 2 * (size_t)(4 + b_boxes) * 128;
  const int rows_target = std::max(8, (int)(budget / 3 / bytes_per_row) / 8 * 8);
  w->npt = std::max(1, rows_target / blk.dim);
  w->rows_pad = (w->npt * blk.dim + 7) / 8 * 8;
  w->stage_bytes = bytes_per_row * (size_t)w->rows_pad;
  w->stages = (int)std::min<size_t>(8, budget / w->stage_bytes);
  if (w->stages < 2) return fail(EQT_ERR_UNSUPPORTED, "irrep with %d components does not fit a reduction tile", blk.dim);
  w->chunk_tiles = std::max(1, 512 / w->rows_pad);
  const int64_t tiles = ceil_div(n, w->npt);
  w->splits = (int)std::max<int64_t>(1, std::min<int64_t>(tiles, sm_count() / w->m_tiles));
  w->need = (int64_t)w->splits * w->m_tiles * 128 * cout;
  return EQT_OK;
}

}  // namespace
}  // namespace eqt

extern "C" int64_t eqt_wgrad_tc_scratch_floats(int64_t n, int32_t cin, int32_t cout, const eqt_mix_block* blocks,
                                               int32_t num_blocks) {
  using namespace eqt;
  if (n < 0 || cin <= 0 || cout <= 0 || cin % 32 || cout % 32 || num_blocks < 0 || (num_blocks && !blocks)) return -1;
  // the sum over the blocks: with that much scratch all blocks run in one launch; eqt_wgrad_tc also works with the
  // largest block's need alone (one launch per block then)
  int64_t need = 0;
  for (int b = 0; b < num_blocks; ++b) {
    WgradShape w{};
    if (wgrad_shape(blocks[b], b, std::max<int64_t>(n, 1), cin, cout, &w)) return -1;
    need += w.need;
  }
  return need;
}

extern "C" int eqt_wgrad_tc(const float* s, const float* g, float* gw_packed, float* scratch, int64_t scratch_floats,
                            int64_t n, int32_t rows, int32_t comps, int32_t cin, int32_t cout,
                            const eqt_mix_block* blocks, int32_t num_blocks, int32_t* status, void* stream) {
  using namespace eqt;
  if (int rc = check_common(s, g, gw_packed, scratch, blocks, status, n, rows, comps, cin, cout, num_blocks))
    return rc < 0 ? EQT_OK : rc;
  if (cin % 32 != 0 || cout % 32 != 0 || cout > 128)
    return fail(EQT_ERR_UNSUPPORTED, "tensor-core weight gradient needs C_in %% 32 == 0, C_out %% 32 == 0, C_out <= 128");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // every block is checked before the first launch, so a refusal leaves gw_packed untouched
  std::vector<WgradShape> shapes(num_blocks);
  for (int b = 0; b < num_blocks; ++b) {
    if (int rc = wgrad_shape(blocks[b], b, n, cin, cout, &shapes[b])) return rc;
    if (shapes[b].need > scratch_floats)
      return fail(EQT_ERR_BAD_ARGUMENT, "scratch too small: block %d needs %lld floats, %lld given", b,
                  (long long)shapes[b].need, (long long)scratch_floats);
  }
  int64_t total_need = 0;
  for (int b = 0; b < num_blocks; ++b) total_need += shapes[b].need;
  // With scratch for every block at once, up to WGRAD_MAX_BLOCKS blocks share a launch (and one reduction launch);
  // otherwise the blocks run one after the other and reuse the scratch.
  const int per_launch = total_need <= scratch_floats ? WGRAD_MAX_BLOCKS : 1;
  for (int b0 = 0; b0 < num_blocks; b0 += per_launch) {
    const int count = std::min(per_launch, num_blocks - b0);
    WgradBatch B{};
    ReduceBatch R{};
    B.count = R.count = count;
    B.n = n; B.n_cols = R.cols = cout; B.status = status;
    B.tmem_cols = 32;
    size_t smem = 0;
    int cta = 0;
    int64_t scratch_at = 0, quads = 0;
    for (int q = 0; q < count; ++q) {
      const eqt_mix_block& blk = blocks[b0 + q];
      const WgradShape& w = shapes[b0 + q];
      WgradBlock& a = B.blk[q];
      a.dim = blk.dim; a.npt = w.npt; a.rows_pad = w.rows_pad; a.stages = w.stages; a.chunk_tiles = w.chunk_tiles;
      a.issuers = w.rows_pad / 8 >= 2 ? 2 : 1;
      a.m_tiles = w.m_tiles; a.splits = w.splits; a.cta_begin = cta;
      a.partial = scratch + scratch_at;
      cta += w.splits * w.m_tiles;
      while (B.tmem_cols < 2 * a.issuers * cout) B.tmem_cols <<= 1;
      smem = std::max(smem, (size_t)w.stages * w.stage_bytes + 1024);
      {
        cuuint64_t dims[3] = {(cuuint64_t)w.K, (cuuint64_t)blk.dim, (cuuint64_t)n};
        cuuint64_t strides[2] = {(cuuint64_t)w.K * 4, (cuuint64_t)rows * cin * 4};
        cuuint32_t box[3] = {KB, (cuuint32_t)blk.dim, (cuuint32_t)w.npt};
        if (int rc = make_map(&a.map_s, s + (int64_t)blk.in_row0 * cin, 3, dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) return rc;
      }
      {
        cuuint64_t dims[3] = {(cuuint64_t)cout, (cuuint64_t)blk.dim, (cuuint64_t)n};
        cuuint64_t strides[2] = {(cuuint64_t)cout * 4, (cuuint64_t)comps * cout * 4};
        cuuint32_t box[3] = {KB, (cuuint32_t)blk.dim, (cuuint32_t)w.npt};
        if (int rc = make_map(&a.map_g, g + (int64_t)blk.out_row0 * cout, 3, dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) return rc;
      }
      R.blk[q].partial = a.partial; R.blk[q].out = gw_packed + blk.w_offset; R.blk[q].splits = w.splits;
      R.blk[q].padded_rows = (int64_t)w.m_tiles * 128; R.blk[q].begin = quads;
      quads += w.K * cout / 4;
      scratch_at += w.need;
    }
    R.total = quads;
    if (int rc = launch_wgrad(B, smem, st)) return rc;
    wgrad_reduce_batched_kernel<<<flat_grid(quads, 256), 256, 0, st>>>(R);
    if (int rc = check_launch("wgrad_reduce_batched_kernel")) return rc;
  }
  return EQT_OK;
}

// ------------------------------------------------------------------------------------------
// The reference's indexed products with shared weights on the same machinery
// ------------------------------------------------------------------------------------------
extern "C" int eqt_vecmat_tc(const float* x, const float* w, const int64_t* index2, const float* scale, float* w_big,
                             float* w_small, float* out, int64_t n, int32_t rows1, int32_t cin, int32_t cout,
                             int32_t num_out, int64_t entries, const int32_t* kb_begin, const int32_t* a_col,
                             int32_t* status, void* stream) {
  using namespace eqt;
  if (n < 0 || rows1 <= 0 || cin <= 0 || cout <= 0 || num_out < 0 || entries < 0) return fail(EQT_ERR_BAD_ARGUMENT, "bad sizes");
  if (n == 0 || num_out == 0) return EQT_OK;
  if (!x || !w || !w_big || !w_small || !out || !kb_begin || !a_col || !status) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  if (cin % KB != 0 || cout % 16 != 0 || cout > 128)
    return fail(EQT_ERR_UNSUPPORTED, "tensor-core vecmat needs C_in %% 32 == 0, C_out %% 16 == 0, C_out <= 128");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(w_big) |
       reinterpret_cast<uintptr_t>(w_small)) & 15u)
    return fail(EQT_ERR_UNSUPPORTED, "tensor-core vecmat needs 16-byte aligned operands");
  if (n > 0x7fffffffll || (int64_t)rows1 * cin > 0x7fffffffll || entries * cin > 0x7fffffffll)
    return fail(EQT_ERR_UNSUPPORTED, "operands too large for one TMA coordinate");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t ktot = entries * cin;
  if (entries > 0) {
    pack_vecmat_weights_kernel<<<flat_grid(ktot * cout, 256), 256, 0, st>>>(w, index2, scale, w_big, w_small, entries, cin, cout);
    if (int rc = check_launch("pack_vecmat_weights_kernel")) return rc;
  }
  VecmatLaunch L{};
  L.out = out; L.kb_begin = kb_begin; L.a_col = a_col; L.n = n; L.num_out = num_out; L.n_cols = cout; L.status = status;
  L.total_items = (int64_t)num_out * ceil_div(n, TILE_M);
  const uint32_t stage_bytes = TILE_M * KB * 4 + 2u * (uint32_t)cout * KB * 4;
  L.stages = (int)std::min<size_t>(std::min<size_t>(8, (220 * 1024 - 1024 - EPI_PATCH_BYTES) / stage_bytes), (512 - 2 * cout) / 64);
  if (L.stages < 2) return fail(EQT_ERR_UNSUPPORTED, "tile too wide for the shared-memory ring");
  L.tmem_cols = 32;
  while (L.tmem_cols < 2 * cout + 64 * L.stages) L.tmem_cols <<= 1;
  {
    cuuint64_t dims[3] = {(cuuint64_t)rows1 * cin, 1, (cuuint64_t)n};
    cuuint64_t strides[2] = {(cuuint64_t)rows1 * cin * 4, (cuuint64_t)rows1 * cin * 4};
    cuuint32_t box[3] = {KB, 1, TILE_M};
    if (int rc = make_map(&L.map_a, x, 3, dims, strides, box)) return rc;
  }
  {
    // an empty table still needs valid maps: describe at least one k-block
    cuuint64_t dims[2] = {(cuuint64_t)std::max<int64_t>(ktot, KB), (cuuint64_t)cout};
    cuuint64_t strides[1] = {(cuuint64_t)std::max<int64_t>(ktot, KB) * 4};
    cuuint32_t box[2] = {KB, (cuuint32_t)cout};
    if (int rc = make_map(&L.map_bb, w_big, 2, dims, strides, box)) return rc;
    if (int rc = make_map(&L.map_bs, w_small, 2, dims, strides, box)) return rc;
  }
  cudaError_t e = cudaFuncSetAttribute(vecmat_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
  if (e != cudaSuccess) return fail(EQT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  const unsigned grid = (unsigned)std::min<int64_t>(L.total_items, sm_count());
  vecmat_tc_kernel<<<grid, TC_THREADS, (size_t)L.stages * stage_bytes + 1024 + EPI_PATCH_BYTES, st>>>(L);
  return check_launch("vecmat_tc_kernel");
}

extern "C" int64_t eqt_outer_tc_scratch_floats(int64_t n, int32_t c2, int32_t m_tiles) {
  using namespace eqt;
  if (n < 0 || c2 <= 0 || c2 % 32 || m_tiles <= 0) return -1;
  const int splits = std::max(1, sm_count() / m_tiles);
  return (int64_t)splits * m_tiles * 128 * c2;
}

extern "C" int eqt_outer_tc(const float* in1, const float* in2, float* out, float* scratch, int64_t scratch_floats, int64_t n,
                            int32_t rows1, int32_t c1, int32_t rows2, int32_t c2, const int32_t* a_cols, const int32_t* b_cols,
                            int32_t m_tiles, const int32_t* red_ptr, const int32_t* red_slot, const float* red_scale,
                            int32_t num_w, int32_t* status, void* stream) {
  using namespace eqt;
  if (n < 0 || rows1 <= 0 || rows2 <= 0 || c1 <= 0 || c2 <= 0 || m_tiles < 0 || num_w < 0) return fail(EQT_ERR_BAD_ARGUMENT, "bad sizes");
  if (num_w == 0) return EQT_OK;
  if (!in1 || !in2 || !out || !scratch || !a_cols || !b_cols || !red_ptr || !red_slot || !red_scale || !status)
    return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  if (c1 % 32 != 0 || c2 % 32 != 0 || c2 > 128)
    return fail(EQT_ERR_UNSUPPORTED, "tensor-core outer product needs C1 %% 32 == 0, C2 %% 32 == 0, C2 <= 128");
  if ((reinterpret_cast<uintptr_t>(in1) | reinterpret_cast<uintptr_t>(in2) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(scratch)) & 15u)
    return fail(EQT_ERR_UNSUPPORTED, "tensor-core outer product needs 16-byte aligned operands");
  if (n > 0x7fffffffll || (int64_t)rows1 * c1 > 0x7fffffffll || (int64_t)rows2 * c2 > 0x7fffffffll)
    return fail(EQT_ERR_UNSUPPORTED, "operands too large for one TMA coordinate");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int splits = 1;
  if (n > 0 && m_tiles > 0) {
    const int b_boxes = c2 / 32;
    const size_t budget = 220 * 1024 - 1024;
    const size_t bytes_per_row = 2 * (size_t)(4 + b_boxes) * 128;
    const int npt = std::max(8, (int)(budget / 3 / bytes_per_row) / 8 * 8);          // reduction rows per tile
    WgradBatch B{};
    B.count = 1; B.n = n; B.n_cols = c2; B.status = status;
    WgradBlock& a = B.blk[0];
    a.dim = 1; a.npt = npt; a.rows_pad = npt;
    const size_t stage_bytes = bytes_per_row * (size_t)npt;
    a.stages = (int)std::min<size_t>(8, budget / stage_bytes);
    a.issuers = npt / 8 >= 2 ? 2 : 1;
    B.tmem_cols = 32;
    while (B.tmem_cols < 2 * a.issuers * c2) B.tmem_cols <<= 1;
    a.chunk_tiles = std::max(1, 512 / npt);
    a.a_cols = a_cols; a.b_cols = b_cols;
    const int64_t tiles = ceil_div(n, npt);
    splits = (int)std::max<int64_t>(1, std::min<int64_t>(tiles, sm_count() / m_tiles));
    const int64_t need = (int64_t)splits * m_tiles * 128 * c2;
    if (need > scratch_floats) return fail(EQT_ERR_BAD_ARGUMENT, "scratch too small: %lld floats needed", (long long)need);
    a.partial = scratch;
    a.m_tiles = m_tiles; a.splits = splits; a.cta_begin = 0;
    {
      cuuint64_t dims[3] = {(cuuint64_t)rows1 * c1, 1, (cuuint64_t)n};
      cuuint64_t strides[2] = {(cuuint64_t)rows1 * c1 * 4, (cuuint64_t)rows1 * c1 * 4};
      cuuint32_t box[3] = {KB, 1, (cuuint32_t)npt};
      if (int rc = make_map(&a.map_s, in1, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) return rc;
    }
    {
      cuuint64_t dims[3] = {(cuuint64_t)rows2 * c2, 1, (cuuint64_t)n};
      cuuint64_t strides[2] = {(cuuint64_t)rows2 * c2 * 4, (cuuint64_t)rows2 * c2 * 4};
      cuuint32_t box[3] = {KB, 1, (cuuint32_t)npt};
      if (int rc = make_map(&a.map_g, in2, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) return rc;
    }
    if (int rc = launch_wgrad(B, (size_t)a.stages * stage_bytes + 1024, st)) return rc;
  }
  // with no samples or no entries every unit list is read as empty only if m_tiles == 0; otherwise the partial sums
  // above were written by this call
  if (n == 0 || m_tiles == 0) {
    cudaError_t e = cudaMemsetAsync(out, 0, sizeof(float) * (size_t)num_w * c1 * c2, st);
    if (e != cudaSuccess) return fail(EQT_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    return EQT_OK;
  }
  outer_reduce_kernel<<<flat_grid((int64_t)num_w * c1 * c2 / 4, 256), 256, 0, st>>>(scratch, out, red_ptr, red_slot, red_scale, splits,
                                                                                   (int64_t)m_tiles * 128, num_w, c1, c2);
  return check_launch("outer_reduce_kernel");
}

// ------------------------------------------------------------------------------------------
// Weight gradient without any caller-side or library-side allocation
// ------------------------------------------------------------------------------------------
namespace eqt {
namespace {

// Scratch for the per-CTA partial sums of eqt_wgrad_tc_static: 148 SMs x 128 rows x 64 columns of
// float32 = 4,849,664 bytes, resident on every GPU that loads this library until the process exits.
constexpr int64_t kStaticScratchFloats = 148ll * 128 * 64;
static __device__ __align__(256) float g_wgrad_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
float* g_static_ptr[kMaxDevices] = {};

// Device address of g_wgrad_scratch on the current device.  In host code the symbol itself is only a
// handle; the address a kernel can use comes from cudaGetSymbolAddress, once per device.
int static_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(EQT_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(EQT_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_wgrad_scratch);
    if (e != cudaSuccess || !p) return fail(EQT_ERR_CUDA, "cudaGetSymbolAddress(g_wgrad_scratch): %s", cudaGetErrorString(e));
    g_static_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_static_ptr[dev];
  return EQT_OK;
}

}  // namespace
}  // namespace eqt

extern "C" int64_t eqt_wgrad_tc_static_capacity(void) { return eqt::kStaticScratchFloats; }

extern "C" int eqt_wgrad_tc_static(const float* s, const float* g, float* gw_packed, int64_t n, int32_t rows,
                                   int32_t comps, int32_t cin, int32_t cout, const eqt_mix_block* blocks,
                                   int32_t num_blocks, int32_t* status, void* stream) {
  using namespace eqt;
  if (cout > 64)
    return fail(EQT_ERR_UNSUPPORTED,
                "eqt_wgrad_tc_static: C_out = %d exceeds the limit of 64 output channels of the built-in scratch "
                "(%lld floats); use eqt_wgrad_tc with a caller-provided scratch buffer", (int)cout,
                (long long)kStaticScratchFloats);
  if ((int64_t)sm_count() * 128 * cout > kStaticScratchFloats)
    return fail(EQT_ERR_UNSUPPORTED,
                "eqt_wgrad_tc_static: %d SMs x 128 x %d floats exceed the built-in scratch of %lld floats; use "
                "eqt_wgrad_tc with a caller-provided scratch buffer", sm_count(), (int)cout,
                (long long)kStaticScratchFloats);
  if (n > 0 && num_blocks > 0 && blocks && cin > 0 && cin % 32 == 0 && cout > 0 && cout % 32 == 0) {
    for (int b = 0; b < num_blocks; ++b) {   // the real need of every block, before anything is launched
      WgradShape w{};
      if (int rc = wgrad_shape(blocks[b], b, n, cin, cout, &w)) return rc;
      if (w.need > kStaticScratchFloats)
        return fail(EQT_ERR_UNSUPPORTED,
                    "eqt_wgrad_tc_static: block %d (%d paths x %d input channels) needs %lld floats of scratch, the "
                    "built-in scratch holds %lld; use eqt_wgrad_tc with a caller-provided scratch buffer", b,
                    (int)blocks[b].paths, (int)cin, (long long)w.need, (long long)kStaticScratchFloats);
    }
  }
  float* scratch = nullptr;
  if (int rc = static_scratch(&scratch)) return rc;
  return eqt_wgrad_tc(s, g, gw_packed, scratch, kStaticScratchFloats, n, rows, comps, cin, cout, blocks, num_blocks,
                      status, stream);
}

// ------------------------------------------------------------------------------------------
// Packing and splitting of the weights for the GEMMs above (one launch instead of a dozen tensor ops)
// ------------------------------------------------------------------------------------------
namespace eqt {
namespace {

struct PackArgs {
  int first[16], paths[16];      // per block: first gathered path, number of paths
  int num_blocks, cin, cout, k_major;
  int64_t total;
};

// k_major = 1: per block Bt[co, p*cin + ci] (operand of eqt_mix_tc);  0: [p*cin + ci, co] (stacked paths)
__global__ void __launch_bounds__(256) pack_weights_kernel(const float* __restrict__ w, const int64_t* __restrict__ gather,
                                                           float* __restrict__ big, float* __restrict__ small, PackArgs a) {
  const int64_t per_path = (int64_t)a.cin * a.cout;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < a.total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t g = i / per_path;              // gathered path this element belongs to (blocks are contiguous runs)
    const int64_t r = i % per_path;
    int ci, co;
    if (a.k_major) {
      int b = 0;
      while (b + 1 < a.num_blocks && g >= a.first[b + 1]) ++b;
      const int64_t local = i - (int64_t)a.first[b] * per_path;      // offset inside the block's (cout, paths*cin) matrix
      const int64_t kk = local % ((int64_t)a.paths[b] * a.cin);
      co = (int)(local / ((int64_t)a.paths[b] * a.cin));
      g = a.first[b] + kk / a.cin;
      ci = (int)(kk % a.cin);
    } else {
      ci = (int)(r / a.cout);
      co = (int)(r % a.cout);
    }
    const float v = __ldg(w + __ldg(gather + g) * per_path + (int64_t)ci * a.cout + co);
    const float hi = rn_tf32(v);
    big[i] = hi;
    small[i] = rn_tf32(v - hi);
  }
}

}  // namespace
}  // namespace eqt

extern "C" int eqt_pack_weights(const float* w, const int64_t* path_gather, int32_t cin, int32_t cout,
                                const eqt_mix_block* blocks, int32_t num_blocks, int32_t k_major, float* big,
                                float* small, void* stream) {
  using namespace eqt;
  if (!w || !path_gather || !blocks || !big || !small) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  if (num_blocks <= 0 || num_blocks > 16 || cin <= 0 || cout <= 0) return fail(EQT_ERR_UNSUPPORTED, "1..16 blocks supported");
  PackArgs a{};
  a.num_blocks = num_blocks; a.cin = cin; a.cout = cout; a.k_major = k_major;
  int total_paths = 0;
  for (int b = 0; b < num_blocks; ++b) {
    a.first[b] = (int)(blocks[b].w_offset / ((int64_t)cin * cout));
    a.paths[b] = blocks[b].paths;
    if (a.first[b] != total_paths) return fail(EQT_ERR_BAD_ARGUMENT, "blocks must be packed back to back");
    total_paths += blocks[b].paths;
  }
  a.total = (int64_t)total_paths * cin * cout;
  pack_weights_kernel<<<flat_grid(a.total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(w, path_gather, big, small, a);
  return check_launch("pack_weights_kernel");
}
