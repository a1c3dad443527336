// Edge featurisation: radius graph over a cell list, and per edge - in the same pass that writes the edge - the
// edge vector, its length, real spherical harmonics, the Bessel radial basis and a cutoff envelope.
//
// The caller bins the points into cubic cells of side >= r (one slab of cells per graph of the batch), sorts them by
// cell and passes the sorted order and the first sorted position of every cell.  One warp owns one target node:
// its lanes walk the points of the 27 surrounding cells, compact the ones closer than r into a list in shared
// memory (ballot + prefix count), and the list is ordered by source index with a rank count so that the result does
// not depend on how the points were binned.  `eqt_radius_count` stores min(#neighbours, max_neighbors) per target;
// after an exclusive scan of those counts `eqt_radius_edges` repeats the search and writes, for the neighbours of
// smallest index, source, target, vec = pos[target] - pos[source], |vec| and the features.
//
// replaces (see include/eqt_b200.h): the chain RadiusGraph -> AddSphericalHarmonics -> AddVectorLengthEmbedding(BesselBasis)
// -> cutoff of the reference's transforms, which calls a third-party neighbour search and then one elementwise
// kernel per operation.
#include <algorithm>

#include "common.cuh"

namespace eqt {
namespace {

#include "generated/sh_specs.inc"

constexpr int RG_WARPS = 4;
constexpr int RG_LIST = 512;        // candidates per target held in shared memory

struct RadiusArgs {
  const float* pos;               // (n, 3)
  const int64_t* batch;           // (n) graph of every point, or NULL
  const int32_t* cell_start;      // (num_cells + 1) into the sorted order
  const int32_t* sorted_index;    // (n) original index of the k-th point in cell order
  const int32_t* point_cell;      // (n) cell of every point (graph slab included), as binned by the caller
  int dims[3];                    // cells per axis (per graph)
  float r2;
  int loop, max_neighbors;
  int64_t n;
  int32_t* degree;                // count pass: (n)
  int32_t* status;                // set to 1 if a target had more than RG_LIST candidates
  // edge pass
  const int64_t* ptr;             // (n + 1)
  int64_t* src;
  int64_t* dst;
  float* vec;                     // (E, 3) or NULL
  float* len;                     // (E) or NULL
  float* sh;                      // (E, (l_max + 1)^2) or NULL
  float* bessel;                  // (E, num_basis) or NULL
  float* cutoff;                  // (E) or NULL
  const float* bessel_w;          // (num_basis) frequencies (n pi by default)
  int l_max, num_basis, cutoff_kind;
  float sh_scale, r_max, cut_min, cut_range, cut_p, cut_eps;
};

// neighbours of target i into list[0 .. count), unsorted; returns the number found (may exceed RG_LIST: the caller flags it)
__device__ __forceinline__ int collect(const RadiusArgs& a, int64_t i, int* list, int lane) {
  const float px = __ldg(a.pos + 3 * i), py = __ldg(a.pos + 3 * i + 1), pz = __ldg(a.pos + 3 * i + 2);
  // the caller's binning is authoritative: the target's cell is read, not recomputed
  const int per_graph = a.dims[0] * a.dims[1] * a.dims[2];
  const int cell = __ldg(a.point_cell + i), local = cell % per_graph;
  const int64_t slab = cell - local;
  const int cx = local % a.dims[0], cy = (local / a.dims[0]) % a.dims[1], cz = local / (a.dims[0] * a.dims[1]);
  int count = 0;
  for (int dz = -1; dz <= 1; ++dz) {
    const int z = cz + dz;
    if (z < 0 || z >= a.dims[2]) continue;
    for (int dy = -1; dy <= 1; ++dy) {
      const int y = cy + dy;
      if (y < 0 || y >= a.dims[1]) continue;
      // the three cells x - 1, x, x + 1 are consecutive in the linear order: one range
      const int x0 = max(cx - 1, 0), x1 = min(cx + 1, a.dims[0] - 1);
      const int64_t c0 = slab + ((int64_t)z * a.dims[1] + y) * a.dims[0] + x0;
      const int k0 = __ldg(a.cell_start + c0), k1 = __ldg(a.cell_start + c0 + (x1 - x0) + 1);
      for (int kb = k0; kb < k1; kb += 32) {
        const int k = kb + lane;
        bool hit = false;
        int j = 0;
        if (k < k1) {
          j = __ldg(a.sorted_index + k);
          const float ex = __ldg(a.pos + 3 * (int64_t)j) - px, ey = __ldg(a.pos + 3 * (int64_t)j + 1) - py,
                      ez = __ldg(a.pos + 3 * (int64_t)j + 2) - pz;
          hit = ex * ex + ey * ey + ez * ez < a.r2 && (a.loop || j != i);
        }
        const unsigned m = __ballot_sync(0xffffffffu, hit);
        if (hit) {
          const int at = count + __popc(m & ((1u << lane) - 1u));
          if (at < RG_LIST) list[at] = j;
        }
        count += __popc(m);
      }
    }
  }
  __syncwarp();
  return count;
}

__global__ void __launch_bounds__(RG_WARPS * 32) radius_count_kernel(RadiusArgs a) {
  __shared__ int lists[RG_WARPS][RG_LIST];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int64_t i = (int64_t)blockIdx.x * RG_WARPS + warp; i < a.n; i += (int64_t)gridDim.x * RG_WARPS) {
    const int count = collect(a, i, lists[warp], lane);
    if (lane == 0) {
      if (count > RG_LIST) atomicExch(a.status, 1);
      a.degree[i] = min(count, a.max_neighbors);
    }
    __syncwarp();
  }
}

template <int LMAX>
__device__ __forceinline__ void write_sh(const RadiusArgs& a, int64_t e, const float (&u)[3]) {
  constexpr int K = (LMAX + 1) * (LMAX + 1);
  float y[K];
  ShUnrolled<float, LMAX>::forward(u, y);
#pragma unroll
  for (int k = 0; k < K; ++k) a.sh[e * K + k] = y[k] * a.sh_scale;
}

__global__ void __launch_bounds__(RG_WARPS * 32) radius_edges_kernel(RadiusArgs a) {
  __shared__ int lists[RG_WARPS][RG_LIST];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int64_t i = (int64_t)blockIdx.x * RG_WARPS + warp; i < a.n; i += (int64_t)gridDim.x * RG_WARPS) {
    const int* list = lists[warp];
    const int count = min(collect(a, i, lists[warp], lane), RG_LIST);
    const int64_t e0 = __ldg(a.ptr + i);
    const int keep = (int)(__ldg(a.ptr + i + 1) - e0);
    const float px = __ldg(a.pos + 3 * i), py = __ldg(a.pos + 3 * i + 1), pz = __ldg(a.pos + 3 * i + 2);
    for (int q = lane; q < count; q += 32) {
      const int j = list[q];
      int rank = 0;
      for (int k = 0; k < count; ++k) rank += list[k] < j;      // sources are distinct
      if (rank >= keep) continue;                               // beyond max_neighbors
      const int64_t e = e0 + rank;
      a.src[e] = j;
      a.dst[e] = i;
      const float vx = px - __ldg(a.pos + 3 * (int64_t)j), vy = py - __ldg(a.pos + 3 * (int64_t)j + 1),
                  vz = pz - __ldg(a.pos + 3 * (int64_t)j + 2);
      const float r = sqrtf(vx * vx + vy * vy + vz * vz);
      if (a.vec) { a.vec[3 * e] = vx; a.vec[3 * e + 1] = vy; a.vec[3 * e + 2] = vz; }
      if (a.len) a.len[e] = r;
      if (a.sh) {
        const float inv = 1.f / fmaxf(r, 1e-12f);
        const float u[3] = {vx * inv, vy * inv, vz * inv};
        switch (a.l_max) {
          case 0: a.sh[e] = a.sh_scale; break;
          case 1: write_sh<1>(a, e, u); break;
          case 2: write_sh<2>(a, e, u); break;
          case 3: write_sh<3>(a, e, u); break;
          default: write_sh<4>(a, e, u); break;
        }
      }
      if (a.bessel) {
        const float pre = 2.f / a.r_max;
        for (int b = 0; b < a.num_basis; ++b) a.bessel[e * a.num_basis + b] = pre * (sinf(__ldg(a.bessel_w + b) * r / a.r_max) / r);
      }
      if (a.cutoff) {
        const float u = fminf(fmaxf((r - a.cut_min) / a.cut_range, 0.f), 1.f);
        float c;
        if (a.cutoff_kind == EQT_CUTOFF_POLYNOMIAL) {
          const float p = a.cut_p;
          c = 1.f - ((p + 1.f) * (p + 2.f) / 2.f) * powf(u, p) + (p * (p + 2.f)) * powf(u, p + 1.f) - (p * (p + 1.f) / 2.f) * powf(u, p + 2.f);
        } else if (a.cutoff_kind == EQT_CUTOFF_COSINE) {
          c = 0.5f * (1.f + cosf(3.14159265358979323846f * u));
        } else {
          c = expf(1.f - 1.f / (1.f - u * u + a.cut_eps));
        }
        a.cutoff[e] = c;
      }
    }
    __syncwarp();
  }
}

int fill_args(const eqt_radius_grid* g, const float* pos, const int64_t* batch, int64_t n, float r, int loop, int max_neighbors,
              int32_t* status, RadiusArgs& a) {
  if (!g || !g->cell_start || !g->sorted_index || !g->point_cell) return fail(EQT_ERR_BAD_ARGUMENT, "incomplete cell list");
  if (n < 0 || r <= 0.f || max_neighbors <= 0) return fail(EQT_ERR_BAD_ARGUMENT, "bad sizes");
  if (g->dims[0] <= 0 || g->dims[1] <= 0 || g->dims[2] <= 0 || !(g->cell_size >= r))
    return fail(EQT_ERR_BAD_ARGUMENT, "cells must be at least r wide");
  if (n > 0x7fffffffll) return fail(EQT_ERR_UNSUPPORTED, "too many points");
  if (n > 0 && (!pos || !status)) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  a.pos = pos; a.batch = batch; a.cell_start = g->cell_start; a.sorted_index = g->sorted_index; a.point_cell = g->point_cell;
  for (int k = 0; k < 3; ++k) a.dims[k] = g->dims[k];
  a.r2 = r * r; a.loop = loop; a.max_neighbors = max_neighbors; a.n = n; a.status = status;
  return EQT_OK;
}

}  // namespace
}  // namespace eqt

extern "C" int eqt_radius_count(const eqt_radius_grid* grid, const float* pos, const int64_t* batch, int64_t n, float r,
                                int32_t loop, int32_t max_neighbors, int32_t* degree, int32_t* status, void* stream) {
  using namespace eqt;
  RadiusArgs a{};
  if (int rc = fill_args(grid, pos, batch, n, r, loop, max_neighbors, status, a)) return rc;
  if (n == 0) return EQT_OK;
  if (!degree) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  a.degree = degree;
  radius_count_kernel<<<flat_grid(ceil_div(n, RG_WARPS), 1, 16), RG_WARPS * 32, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return check_launch("radius_count_kernel");
}

extern "C" int eqt_radius_edges(const eqt_radius_grid* grid, const float* pos, const int64_t* batch, int64_t n, float r,
                                int32_t loop, int32_t max_neighbors, const int64_t* ptr, int64_t* src, int64_t* dst,
                                const eqt_edge_features* f, int32_t* status, void* stream) {
  using namespace eqt;
  RadiusArgs a{};
  if (int rc = fill_args(grid, pos, batch, n, r, loop, max_neighbors, status, a)) return rc;
  if (n == 0) return EQT_OK;
  if (!ptr || !src || !dst) return fail(EQT_ERR_BAD_ARGUMENT, "NULL pointer");
  a.ptr = ptr; a.src = src; a.dst = dst;
  if (f) {
    if (f->sh && (f->l_max < 0 || f->l_max > 4)) return fail(EQT_ERR_UNSUPPORTED, "fused harmonics take l_max <= 4");
    if (f->bessel && (!f->bessel_weights || f->num_basis <= 0 || !(f->r_max > 0.f))) return fail(EQT_ERR_BAD_ARGUMENT, "bad radial basis");
    if (f->cutoff && (f->cutoff_kind < EQT_CUTOFF_POLYNOMIAL || f->cutoff_kind > EQT_CUTOFF_MOLLIFIER || !(f->cutoff_r_max > f->cutoff_r_min)))
      return fail(EQT_ERR_BAD_ARGUMENT, "bad cutoff");
    a.vec = f->vec; a.len = f->length; a.sh = f->sh; a.bessel = f->bessel; a.cutoff = f->cutoff; a.bessel_w = f->bessel_weights;
    a.l_max = f->l_max; a.num_basis = f->num_basis; a.cutoff_kind = f->cutoff_kind;
    a.sh_scale = f->integral_normalize ? 0.28209479177387814f : 1.f;
    a.r_max = f->r_max; a.cut_min = f->cutoff_r_min; a.cut_range = f->cutoff_r_max - f->cutoff_r_min;
    a.cut_p = f->cutoff_p; a.cut_eps = f->cutoff_eps;
  }
  radius_edges_kernel<<<flat_grid(ceil_div(n, RG_WARPS), 1, 16), RG_WARPS * 32, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return check_launch("radius_edges_kernel");
}
