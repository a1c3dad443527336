/*
 * eqt_b200: C ABI of the sm_100a kernels behind Equitorch's sparse tensor-product path.
 *
 * Every entry point takes plain device pointers and sizes, launches on the given CUDA
 * stream (a cudaStream_t passed as void*; NULL = legacy default stream), never
 * synchronises, never allocates (except where stated) and returns 0 or an EQT_ERR_* code.
 * eqt_last_error() returns a static description of the most recent failure of the
 * calling thread.  Index arrays are int64 on the device, exactly as the reference's
 * Info tuples hold them; a NULL index array means "identity" (0, 1, 2, ...).
 *
 * The "replaces" notes name the reference interface each entry point stands in for
 * (paths relative to the reference repository root).
 */
#ifndef EQT_B200_H
#define EQT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum eqt_status {
  EQT_OK = 0,
  EQT_ERR_BAD_ARGUMENT = 1,   /* NULL pointer, negative size, unknown enum value            */
  EQT_ERR_UNSUPPORTED = 2,    /* valid request that no kernel covers (e.g. size limits)     */
  EQT_ERR_CUDA = 3            /* a CUDA runtime call failed; see eqt_last_error()           */
};

enum eqt_dtype { EQT_F32 = 0, EQT_F64 = 1, EQT_BF16 = 2 };

/* Which pairwise product is formed for each table entry. */
enum eqt_op {
  EQT_OP_MUL = 0,     /* x[.., c]   * y[.., c]                    -> (.., c)       */
  EQT_OP_VECSCA = 1,  /* x[.., c]   * y[..]   (y has no channel)   -> (.., c)       */
  EQT_OP_SCALE = 2,   /* x[.., c]             (no second operand)  -> (.., c)       */
  EQT_OP_OUTER = 3,   /* x[.., c1]  * y[.., c2]                    -> (.., c1, c2)  */
  EQT_OP_INNER = 4,   /* sum_c x[.., c] * y[.., c]                 -> (..)          */
  EQT_OP_VECMAT = 5   /* sum_ci x[.., ci] * y[.., ci, co]          -> (.., co)      */
};

/*
 * out[n, index_out[o] | o, ...] = sum_{t in [seg[o], seg[o+1])}  scale[t'] * in1[n | -, index1[t'], ..] (op) in2[n | -, index2[t'], ..]
 * with t' = gather_index[t] (or t).  Without seg there is one entry per computed row (t = o).
 * With `accumulated` the batch dimension n is summed away and `out` has no batch dimension.
 *
 * Layouts are contiguous row-major: in1 (n | 1, rows1, c1), in2 per op (see eqt_op),
 * out (n, out_size, ...) or (out_size, ...) when accumulated.  `out` must be zero-filled by
 * the caller when `accumulated` or `index_out` is used; otherwise rows [0, num_out) are
 * fully overwritten (an empty segment writes zeros).
 * dtype is the element type of in1, in2 and of a non-accumulated out.  Sums are carried in
 * float (double for EQT_F64) whatever the storage type; `scale` and an accumulated out have that
 * arithmetic type (float for EQT_F32 / EQT_BF16, double for EQT_F64).
 */
typedef struct eqt_product_args {
  int32_t op;            /* enum eqt_op                                             */
  int32_t dtype;         /* enum eqt_dtype                                          */
  int32_t shared1;       /* in1 has no batch dimension                              */
  int32_t shared2;       /* in2 has no batch dimension                              */
  int32_t accumulated;   /* sum over the batch                                      */
  int32_t reserved;
  const void* in1;
  const void* in2;       /* NULL for EQT_OP_SCALE                                   */
  void* out;
  const void* scale;     /* (T,) float | double (see above), or NULL (= 1)         */
  const int64_t* index1; /* (T,) rows of in1, or NULL                               */
  const int64_t* index2; /* (T,) rows of in2, or NULL                               */
  const int64_t* seg;    /* (num_out + 1,) CSR pointer into the table, or NULL      */
  const int64_t* gather_index; /* (seg[num_out],) indirection into the table, or NULL */
  const int64_t* index_out;    /* (num_out,) output row of each computed row, or NULL */
  int64_t n;             /* batch size                                              */
  int64_t rows1;         /* sparse extent of in1                                    */
  int64_t rows2;         /* sparse extent of in2                                    */
  int64_t num_out;       /* computed rows                                           */
  int64_t out_size;      /* rows of the output tensor (>= num_out unless scattered) */
  int64_t c1;            /* channels of in1 (reduction size for INNER / VECMAT)     */
  int64_t c2;            /* OUTER: channels of in2; VECMAT: output channels; else 0 */
} eqt_product_args;

/*
 * Generic batched sparse-dense product.
 * replaces: equitorch/ops/batched_sparse_dense_op.py
 *   indexed_mul_scale_gather :277, indexed_outer_scale_gather :557, indexed_inner_scale_gather :833,
 *   indexed_vecmat_scale_gather :1511, indexed_vecsca_scale_gather :1796 (and the argument-swapping
 *   aliases indexed_scavec_scale_gather :994, indexed_mat_t_vec_scale_gather :1200), and
 *   equitorch/ops/indexed_scale_segment_op.py indexed_scale_segment :172 (EQT_OP_SCALE).
 */
int eqt_sparse_product(const eqt_product_args* args, void* stream);

/*
 * Real spherical harmonics by the degree recurrence
 *   Y_l[m] = sum_e coef[e] * xyz[axis[e]] * Y_{l-1}[m_in[e]],   Y_0 = 1,
 * entries of degree l stored in [ptr[l], ptr[l+1]) with m_out ascending.
 * xyz (n, 3), out (n, (l_max+1)^2), same dtype (EQT_F32 or EQT_F64).  With `normalize` the
 * vector is divided by max(|v|, 1e-12) first; `out_scale` multiplies every component.
 * replaces: equitorch/ops/spherical_harmonics.py spherical_harmonics :69 plus the
 *   normalisation of equitorch/nn/sphericals.py :31-35.
 */
typedef struct eqt_sh_table {
  const int32_t* ptr;    /* (l_max + 2,) device, ptr[0] = ptr[1] = 0                */
  const int32_t* m_out;  /* (E,) device, component within degree l                  */
  const int32_t* m_in;   /* (E,) device, component within degree l-1                */
  const int32_t* axis;   /* (E,) device, 0 = x, 1 = y, 2 = z                        */
  const double* coef;    /* (E,) device                                             */
  int32_t l_max;
  int32_t num_entries;
} eqt_sh_table;

int eqt_sh_forward(int32_t dtype, const void* xyz, void* out, int64_t n, const eqt_sh_table* table,
                   int32_t normalize, double out_scale, void* stream);

/* grad_xyz (n, 3) = d(sum out * grad_out)/d xyz, through the normalisation when enabled. */
int eqt_sh_backward(int32_t dtype, const void* xyz, const void* grad_out, void* grad_xyz, int64_t n,
                    const eqt_sh_table* table, int32_t normalize, double out_scale, void* stream);

/*
 * Rows of a node tensor summed over CSR segments of (sorted) edges, and the matching gather.
 *   eqt_segment_sum: out[d, :] = sum_{e in [ptr[d], ptr[d+1])} in[perm[e] | e, :]
 *   eqt_gather_rows: out[e, :] = in[index[e], :]
 * width = elements per row; dtype EQT_F32 / EQT_F64 / EQT_BF16 (sums carried in float).
 * replaces: the torch_geometric.utils.scatter / segment call and the edge_index gather a user of
 *   the reference places around the layer (equitorch/transforms/__init__.py :99-101 shows the
 *   edge_index[0] = source, edge_index[1] = destination convention).
 */
int eqt_segment_sum(int32_t dtype, const void* in, const int64_t* ptr, const int64_t* perm, void* out,
                    int64_t num_segments, int64_t width, void* stream);
int eqt_gather_rows(int32_t dtype, const void* in, const int64_t* index, void* out, int64_t num_rows,
                    int64_t width, void* stream);

/*
 * CG step of a tensor-product layer whose second operand has no channel axis, for one role
 * assignment: table entry t adds  scale[t] * feat[.., m_feat[t], c] * y[.., m_y[t]]  to intermediate
 * row r, where the entries of row r are [row_ptr[r], row_ptr[r+1]).  These are the fields of the
 * reference's SparseProductInfo `info_Mij_fwd` (equitorch/structs/__init__.py:67-81, built by
 * equitorch/utils/_structs.py:219-227) with the segment pointer kept and the operand roles named.
 * `structure_key` identifies index structures whose inner loops were unrolled at build time
 * (0 = unknown: the table-driven kernels are used).
 */
typedef struct eqt_tp_table {
  const float* scale;       /* (T,) device                                            */
  const int64_t* m_feat;    /* (T,) component of the channelled operand               */
  const int64_t* m_y;       /* (T,) component of the channel-less operand             */
  const int64_t* row_ptr;   /* (R + 1,)                                               */
  int32_t num_entries;      /* T                                                      */
  int32_t num_rows;         /* R                                                      */
  int32_t d_feat;           /* components of the channelled operand                   */
  int32_t d_y;              /* components of the channel-less operand (<= 255)        */
  uint64_t structure_key;
  const float* scale_o;     /* scale permuted into the unrolled kernels' role order (zero padded; see
                               gen_tp_specs.outer_order), or NULL (then only table-driven kernels run) */
} eqt_tp_table;

/*
 * Gather, CG contraction and sum over the edges of each output node in one pass (float32):
 *   out[d, r, c] = sum_{e in [seg_ptr[d], seg_ptr[d+1])} sum_{t in row r}
 *                      scale[t] * y[y_index[e] | e, m_y[t]] * feat[feat_index[e] | e, m_feat[t], c]
 * feat (rows, d_feat, channels), y (.., d_y), out (num_out, R, channels).  seg_ptr == NULL means one
 * edge per output row (num_out == num_edges, no reduction): the plain per-sample CG step.
 * `status` points to a device int that is set to 1 if a bounded wait inside the kernel gave up.
 * replaces: the chain  x[edge_index[0]] -> indexed_vecsca_scale_gather (equitorch/ops/
 *   batched_sparse_dense_op.py:1796, called from equitorch/nn/functional/linears.py:262) ->
 *   torch_geometric scatter-sum over edge_index[1]; with the roles of the backward-1 tables it is
 *   the scavec step of tensor_product_1vu (linears.py:341-363) summed over edge sources.
 */
int eqt_tp_cg_segment_sum(const eqt_tp_table* table, const float* feat, const int64_t* feat_index,
                          const float* y, const int64_t* y_index, const int64_t* seg_ptr, float* out,
                          int64_t num_out, int64_t num_edges, int32_t channels, int32_t* status, void* stream);

/*
 * Adjoint of the CG step with respect to the channel-less operand (float32):
 *   grad_y[y_index[e] | e, k] = sum_{t: m_y[t] = k} scale[t] * sum_c feat[feat_index[e] | e, m_feat[t], c] * g[node(e), row(t), c]
 * g (num_nodes, R, channels) holds the gradient with respect to the intermediate, already summed
 * per node; edges are sorted by node (seg_ptr, and edge_node for the table-driven kernel).
 * replaces: indexed_inner_scale_gather on the `info_Mij_bwd2` table (equitorch/nn/functional/
 *   linears.py:308-311) fed with per-edge copies of g.
 */
int eqt_tp_cg_inner(const eqt_tp_table* table, const float* feat, const int64_t* feat_index, const float* g,
                    const int64_t* seg_ptr, const int64_t* edge_node, const int64_t* y_index, float* grad_y,
                    int64_t num_nodes, int64_t num_edges, int32_t channels, int32_t* status, void* stream);

/*
 * Weight step of a layer with weights shared by all samples, on tensor cores (float32 in and out,
 * 3xTF32 split arithmetic, accumulation in float32):
 *   out[i, out_row0 + m, co] = sum_{p < paths} sum_ci s[i, in_row0 + m*paths + p, ci] * W_p[ci, co]
 * for every block (= output irrep) and m < dim.  s (n, rows, cin), out (n, comps, cout).  The
 * weights of a block are passed packed and split: w_big / w_small + w_offset point to a (cout, paths*cin)
 * row-major matrix Bt[co, p*cin + ci] = W_p[ci, co], with w_big = W rounded to TF32 (10 mantissa
 * bits) and w_small = (W - w_big) rounded to TF32.  `blocks` is a host array.  Needs cin % 32 == 0, cout % 16 == 0,
 * cout <= 256 and 16-byte aligned pointers, else EQT_ERR_UNSUPPORTED (callers then use
 * eqt_sparse_product with EQT_OP_VECMAT).  `status` is set to 2 if a bounded wait expired.
 * replaces: indexed_vecmat_scale_gather (equitorch/ops/batched_sparse_dense_op.py:1511) as called by
 *   sparse_vecmat on the `info_M_fwd` table (equitorch/nn/functional/linears.py:263).
 */
typedef struct eqt_mix_block {
  int32_t in_row0;    /* first intermediate row of the block (its dim*paths rows are contiguous) */
  int32_t out_row0;   /* first output component of the block                                     */
  int32_t dim;        /* components of the output irrep (<= 128)                                  */
  int32_t paths;      /* paths coupling into it                                                   */
  int64_t w_offset;   /* offset in floats of the block's packed weights                           */
} eqt_mix_block;

int eqt_mix_tc(const float* s, const float* w_big, const float* w_small, float* out, int64_t n, int32_t rows,
               int32_t comps, int32_t cin, int32_t cout, const eqt_mix_block* blocks, int32_t num_blocks,
               int32_t* status, void* stream);

/*
 * Adjoint of the weight step with respect to the intermediate, same arithmetic:
 *   g_inter[i, in_row0 + m*paths + p, ci] = sum_co g[i, out_row0 + m, co] * W_p[ci, co]
 * g (n, comps, cout), g_inter (n, rows, cin).  Here w_big / w_small + w_offset point to the block's
 * (paths*cin, cout) row-major matrix B[p*cin + ci, co] = W_p[ci, co] (the weights of the block's paths
 * stacked, no transpose), split like above; w_offset is in floats as before (paths*cin*cout per block).
 * Needs cout % 32 == 0, cin % 16 == 0, cin <= 256.
 * replaces: indexed_mat_t_vec_scale_gather on the `info_M_bwd1` table, the gradient of sparse_vecmat
 *   with respect to its vector input (equitorch/nn/functional/sparse_product.py:268-270).
 */
int eqt_mix_tc_transposed(const float* g, const float* w_big, const float* w_small, float* g_inter, int64_t n,
                          int32_t rows, int32_t comps, int32_t cin, int32_t cout, const eqt_mix_block* blocks,
                          int32_t num_blocks, int32_t* status, void* stream);

/*
 * Gradient of the weight step with respect to weights shared by all samples, on tensor cores:
 *   gw_packed[w_offset + (p*cin + ci)*cout + co] = sum_i sum_m s[i, in_row0 + m*paths + p, ci] * g[i, out_row0 + m, co]
 * i.e. per block a (paths*cin, cout) row-major matrix, the same stacking as the weights handed to
 * eqt_mix_tc_transposed.  The sum over the n samples is split over CTAs; their float32 partial sums go
 * through `scratch` (caller-owned, contents undefined afterwards) and are reduced in a fixed order: no atomics,
 * results are bit-reproducible.  A block needs 128 * cout * #SMs floats of scratch (more only with over
 * 128 * #SMs stacked input channels).  With eqt_wgrad_tc_scratch_floats(...) floats - the sum over the blocks -
 * all blocks run in one launch; with at least the largest block's need they run one launch per block and share
 * the scratch; the results are the same bit for bit.  All blocks are checked before the first launch: an error
 * return leaves gw_packed untouched.
 * Needs cin % 32 == 0, cout % 32 == 0, cout <= 128.
 * replaces: indexed_outer_scale_gather with out_accumulated=True on the `info_M_bwd2` table
 *   (equitorch/nn/functional/linears.py:316-320), which uses atomic adds in the reference.
 */
int eqt_wgrad_tc(const float* s, const float* g, float* gw_packed, float* scratch, int64_t scratch_floats, int64_t n,
                 int32_t rows, int32_t comps, int32_t cin, int32_t cout, const eqt_mix_block* blocks,
                 int32_t num_blocks, int32_t* status, void* stream);
/* Floats of scratch with which eqt_wgrad_tc runs these blocks in one launch on the current device (the sum of the
 * blocks' needs), or -1 for blocks it refuses (host-side arithmetic only; part of the eqt_wgrad_tc interface above). */
int64_t eqt_wgrad_tc_scratch_floats(int64_t n, int32_t cin, int32_t cout, const eqt_mix_block* blocks, int32_t num_blocks);

/*
 * The reference's indexed vector-matrix product with weights shared by the batch, on tensor cores (float32, 3xTF32):
 *   out[i, M, co] = sum_{t in seg[M]} scale[t] * sum_ci x[i, index1[t], ci] * W[index2[t], ci, co]
 * x (n, rows1, cin), W (.., cin, cout), out (n, num_out, cout).  Per output row M the entries of seg[M] form one
 * GEMM over the samples whose k-blocks are 32-channel chunks of x rows; `kb_begin` (num_out + 1, device int32) is
 * seg scaled to k-blocks (seg[M] * cin / 32) and `a_col` (entries * cin / 32, device int32) the column
 * index1[t] * cin + 32 * chunk each k-block starts at - both depend on the table only and are built once.
 * The weights are packed as Bt[co, t * cin + ci] = scale[t] * W[index2[t], ci, co] and split into TF32 big / small
 * parts by this call into w_big / w_small (entries * cin * cout floats each, caller-owned scratch).  index2 / scale
 * may be NULL (identity / ones).  Needs cin % 32 == 0, cout % 16 == 0, cout <= 128, 16-byte aligned pointers.
 * `status` is set to 2 if a bounded wait expired.
 * replaces: indexed_vecmat_scale_gather (equitorch/ops/batched_sparse_dense_op.py:1511-1534, kernel :1289-1381) for
 *   a 3-D (shared) matrix operand, i.e. SO2Linear, IrrepWiseLinear, IrrepsLinear and the weight step of SO3Linear
 *   'uv' (equitorch/nn/functional/linears.py:494-577, :263) and their input gradients.
 */
int eqt_vecmat_tc(const float* x, const float* w, const int64_t* index2, const float* scale, float* w_big,
                  float* w_small, float* out, int64_t n, int32_t rows1, int32_t cin, int32_t cout, int32_t num_out,
                  int64_t entries, const int32_t* kb_begin, const int32_t* a_col, int32_t* status, void* stream);

/*
 * The reference's indexed outer product accumulated over the batch (the gradient of shared weights), on tensor
 * cores, deterministic:
 *   out[w, a, b] = sum_i sum_{t in seg[w]} scale[t] * in1[i, index1[t], a] * in2[i, index2[t], b]
 * in1 (n, rows1, c1), in2 (n, rows2, c2), out (num_w, c1, c2).  A "unit" is a 32-column chunk of an in1 row of
 * one entry; units that share their in2 row are packed four to an M slice of 128 rows: a_cols (m_tiles * 4) holds
 * the first in1 column of every slot (any valid column for padding slots), b_cols (m_tiles) the first in2 column of
 * the slice.  Every CTA reduces a share of the samples for one slice on tcgen05 (TF32 big / small split, TMEM folded
 * into float32 registers every ~512 samples); the per-CTA sums go through `scratch`
 * (eqt_outer_tc_scratch_floats(n, c2, m_tiles) floats) and are combined in a fixed order:
 * out[w, ci, :] = sum over the units u in [red_ptr[w * c1/32 + ci/32], red_ptr[.. + 1]) of red_scale[u] * (row
 * red_slot[u] * 32 + ci % 32 of the summed slices).  No atomics.  Needs c1 % 32 == 0, c2 % 32 == 0, c2 <= 128.
 * replaces: indexed_outer_scale_gather with out_accumulated=True (equitorch/ops/batched_sparse_dense_op.py:557-579,
 *   kernel :343-434, which adds 32 x 32 tiles with tl.atomic_add).
 */
int eqt_outer_tc(const float* in1, const float* in2, float* out, float* scratch, int64_t scratch_floats, int64_t n,
                 int32_t rows1, int32_t c1, int32_t rows2, int32_t c2, const int32_t* a_cols, const int32_t* b_cols,
                 int32_t m_tiles, const int32_t* red_ptr, const int32_t* red_slot, const float* red_scale,
                 int32_t num_w, int32_t* status, void* stream);
int64_t eqt_outer_tc_scratch_floats(int64_t n, int32_t c2, int32_t m_tiles);

/*
 * eqt_wgrad_tc for callers that cannot hand over a scratch buffer because they cannot allocate device
 * memory at the point of the call: a C or Fortran host program that links this library without a
 * CUDA allocator of its own, or a plug-in running inside a framework that reserved all device memory
 * in its own arena at start-up and forbids cudaMalloc afterwards.  Same arguments and results as
 * eqt_wgrad_tc minus `scratch`; the per-CTA partial sums go through a 4.85 MB array that is part of the
 * library image on every GPU (148 x 128 x 64 floats, eqt_wgrad_tc_static_capacity()).  The function
 * and everything it calls allocate nothing.
 *   - Limit: cout <= 64 and every block's own need (#SMs * 128 * cout for ordinary layers) must fit the array
 *     (the blocks run one launch each and share it); larger requests return EQT_ERR_UNSUPPORTED with a message naming the limit, before
 *     anything is launched - use eqt_wgrad_tc then.
 *   - The first call on each device looks up the array's device address (with that device current);
 *     make that first call outside any stream capture.
 *   - All calls on a device share the one array.  Nothing in it has to be zero on entry (every partial
 *     sum that is read back was written by the same call), but two calls whose kernels overlap on the
 *     GPU (different streams) race on it: serialise them.
 * No counterpart in the reference: it has no C interface and leaves all allocation to PyTorch.
 */
int eqt_wgrad_tc_static(const float* s, const float* g, float* gw_packed, int64_t n, int32_t rows, int32_t comps,
                        int32_t cin, int32_t cout, const eqt_mix_block* blocks, int32_t num_blocks,
                        int32_t* status, void* stream);
int64_t eqt_wgrad_tc_static_capacity(void);

/*
 * Gather, lay out and split shared weights w (num_paths, cin, cout) for the tensor-core entry points:
 * path_gather (device, int64) lists the paths of all blocks back to back (w_offset of a block =
 * first gathered path * cin * cout).  k_major != 0 writes the per-block (cout, paths*cin) matrices that
 * eqt_mix_tc reads, k_major == 0 the stacked (paths*cin, cout) matrices of eqt_mix_tc_transposed;
 * big = TF32-rounded value, small = TF32-rounded remainder.  No counterpart in the reference.
 */
int eqt_pack_weights(const float* w, const int64_t* path_gather, int32_t cin, int32_t cout, const eqt_mix_block* blocks,
                     int32_t num_blocks, int32_t k_major, float* big, float* small, void* stream);

/* Library / device facts. */
const char* eqt_last_error(void);
int eqt_version(void);
/* Kernel launches issued by this library in the calling process since load (for benchmarks). */
int64_t eqt_launch_count(void);

/*
 * Per-irrep streaming kernels behind Gate, the norms and the RMS normalisations (float32 / float64).
 *   eqt_irrep_scale: out[n, i, c] = x[n, i, c] * s(n, irrep_index[i], c); s_mode 0: s is (n, k, c), 1: s is (k, c)
 *                    shared by all samples, 2: s is (n, k), one scalar per sample and irrep.
 *                    replaces: gating, equitorch/nn/functional/activations.py:31-36, and the scaling steps of
 *                    batch_rms_norm / layer_rms_norm, equitorch/nn/functional/normalization.py:58-63,147-156
 *                    (sparse_mul / sparse_vecsca with index2 = irrep_index).
 *   eqt_irrep_dot:   out[n, kk, c] = sum_{i in [irrep_seg[kk], irrep_seg[kk+1])} a[n, i, c] * b[n, i, c]; a == b
 *                    gives the squared norms.  replaces: segment(input.pow(2), irrep_seg),
 *                    equitorch/nn/functional/norm.py:26,75,143,206, and the gate-gradient reduction
 *                    (sparse_mul with seg_out = irrep_seg).
 * x / a / b are (n, d, c) contiguous, d <= 1024 components in k irreps.
 */
int eqt_irrep_scale(const void* x, const void* s, void* out, const int64_t* irrep_index, int64_t n, int32_t d,
                    int32_t k, int32_t c, int32_t s_mode, int32_t dtype, void* stream);
int eqt_irrep_dot(const void* a, const void* b, void* out, const int64_t* irrep_seg, int64_t n, int32_t d,
                  int32_t k, int32_t c, int32_t dtype, void* stream);

/*
 * Fused LayerRMSNorm (float32 / float64): per sample n and irrep k
 *   rsigma[n, k] = (mean_c sum_{i in k} x[n, i, c]^2 (/ dim_k if scaled) + eps)^-1/2
 *   out[n, i, c] = x[n, i, c] * rsigma[n, k(i)] * weight[k(i), c]            (weight may be NULL)
 * in one pass (one warp per sample), and its backward: grad_x, plus per-warp partial sums of grad_weight,
 * grad_weight_partial (eqt_layer_rms_num_partials(n), k, c), which the caller sums over the first dimension
 * (NULL = not wanted).  Needs k <= 16, C / 4 (float32) or C / 2 (float64) dividing 32, 16-byte aligned tensors;
 * EQT_ERR_UNSUPPORTED otherwise.
 * replaces: layer_rms_norm, equitorch/nn/functional/normalization.py:112-160 (channel_mean_squared_norm,
 * sparse_vecsca, sparse_mul and their backward passes).
 */
int eqt_layer_rms_num_partials(int64_t n);
int eqt_layer_rms_forward(const void* x, const void* weight, void* out, void* rsigma, const int64_t* irrep_seg,
                          int64_t n, int32_t d, int32_t k, int32_t c, int32_t scaled, double eps, int32_t dtype,
                          void* stream);
int eqt_layer_rms_backward(const void* x, const void* grad_out, const void* weight, const void* rsigma, void* grad_x,
                           void* grad_weight_partial, const int64_t* irrep_seg, int64_t n, int32_t d, int32_t k,
                           int32_t c, int32_t scaled, int32_t dtype, void* stream);

/*
 * Wigner-D matrices of ZYZ Euler angles,  D = Z(alpha) J Z(beta) J Z(gamma)  per irrep block (real basis, component
 * order m = -l..l, Z(a): x'_m = cos(m a) x_m - sign(m) sin(|m| a) x_{-m}), written as a dense block-diagonal
 * (n, dim, dim) tensor in one pass, and the gradient of a scalar with respect to the three angles from grad_d
 * (only the in-block elements of grad_d are read).  The table holds, per irrep block of degree l, the coefficients
 * of the trigonometric polynomial  J Z(beta) J = sum_k A_k cos(k beta) + B_k sin(k beta):  (l + 1) x (2l+1) x (2l+1) x 2
 * values [k][a][b][A, B] in the dtype of the call.  float32 / float64, degrees up to 7.
 * replaces: wigner_d_matrix (equitorch/nn/functional/wigner_d.py:74-139: sincos :4-35 of nn/functional/angular.py,
 *   three sparse_vecsca z-rotations and two sparse_scale J passes over the identity) and its autograd chain.
 */
typedef struct eqt_wigner_table {
  const void* coef;        /* device, coef_count values                                                  */
  const int32_t* comp;     /* device (dim, 4): first component of the block, l, coefficient offset, m    */
  const int32_t* blocks;   /* device (num_blocks, 3): first component, l, coefficient offset             */
  int32_t dim, num_blocks, max_l, coef_count;
} eqt_wigner_table;
int eqt_wigner_d_forward(const eqt_wigner_table* table, const void* alpha, const void* beta, const void* gamma, void* d,
                         int64_t n, int32_t dtype, void* stream);
int eqt_wigner_d_backward(const eqt_wigner_table* table, const void* alpha, const void* beta, const void* gamma,
                          const void* grad_d, void* grad_alpha, void* grad_beta, void* grad_gamma, int64_t n,
                          int32_t dtype, void* stream);

/*
 * Dense rotation of features by a per-sample matrix:  out[n, i, c] = sum_j matrix[n, i, j] x[n, j, c]  (with
 * `transposed`: matrix[n, j, i]), matrix (n, dim, dim), x / out (n, dim, channels), and the gradient with respect
 * to the matrix, grad_matrix[n, i, j] = sum_c grad_out[n, i, c] x[n, j, c].  float32 / float64.
 * replaces: dense_wigner_rotation = `wigner_d @ input` (equitorch/nn/functional/wigner_d.py:58-72,
 *   equitorch/nn/wigner_d.py:89-106) and the two batched products of its backward pass.
 * row_range (optional, device, dim x 2 int32): for matrices that are block diagonal over irreps, the column range
 *   [lo, hi) of every row's block.  Only those entries of `matrix` are read and multiplied, and grad_matrix is zero
 *   outside them.  NULL = dense.
 */
int eqt_dense_rotation(const void* matrix, const void* x, void* out, int64_t n, int32_t dim, int32_t channels,
                       int32_t transposed, const int32_t* row_range, int32_t dtype, void* stream);
int eqt_dense_rotation_grad_matrix(const void* grad_out, const void* x, void* grad_matrix, int64_t n, int32_t dim,
                                   int32_t channels, const int32_t* row_range, int32_t dtype, void* stream);

/*
 * Radius graph and edge features in one pass over a cell list (float32).
 * The caller bins the n points into cubic cells of side cell_size >= r - `dims` cells per axis, x fastest:
 * cell = ((graph * dims[2] + z) * dims[1] + y) * dims[0] + x, one slab of cells per graph of the batch - and
 * passes point_cell (n), the points' indices sorted by cell (sorted_index) and the first sorted position of every
 * cell (cell_start, number of cells + 1), all int32 on the device.
 * eqt_radius_count: degree[i] = min(#{j : |pos_i - pos_j| < r, same graph, j != i unless loop}, max_neighbors).
 * eqt_radius_edges: with ptr = exclusive scan of degree (n + 1, int64), for every target i the max_neighbors
 * neighbours of smallest index j, ascending, at e = ptr[i] + rank: src[e] = j, dst[e] = i and, where the pointer in
 * `features` is not NULL,
 *   vec[e]    = pos[i] - pos[j]                       length[e] = |vec[e]|
 *   sh[e, :]  = real spherical harmonics of vec / max(|vec|, 1e-12), l <= l_max <= 4, component normalised
 *               (times 1 / sqrt(4 pi) with integral_normalize)
 *   bessel[e, b] = (2 / r_max) sin(bessel_weights[b] |vec| / r_max) / |vec|
 *   cutoff[e] = polynomial (p) / cosine / mollifier (eps) envelope of u = clamp((|vec| - r_min) / (r_max - r_min), 0, 1)
 * `status` is set to 1 if a target had more than 512 candidates (its list is then truncated).
 * replaces: RadiusGraph, AddVectorNorm, AddSphericalHarmonics, AddVectorLengthEmbedding
 *   (equitorch/transforms/__init__.py:18-251; the neighbour search itself is torch_geometric.nn.radius_graph, not
 *   part of the reference's sources), BesselBasis (equitorch/nn/radials.py:10-56) and the cutoffs
 *   (equitorch/nn/functional/cutoffs.py).
 */
enum eqt_cutoff_kind { EQT_CUTOFF_POLYNOMIAL = 0, EQT_CUTOFF_COSINE = 1, EQT_CUTOFF_MOLLIFIER = 2 };
typedef struct eqt_radius_grid {
  const int32_t* cell_start;
  const int32_t* sorted_index;
  const int32_t* point_cell;
  float cell_size;
  int32_t dims[3];
} eqt_radius_grid;
typedef struct eqt_edge_features {
  float* vec;                    /* (E, 3) or NULL                  */
  float* length;                 /* (E) or NULL                     */
  float* sh;                     /* (E, (l_max + 1)^2) or NULL      */
  float* bessel;                 /* (E, num_basis) or NULL          */
  float* cutoff;                 /* (E) or NULL                     */
  const float* bessel_weights;   /* (num_basis) device              */
  int32_t l_max, integral_normalize, num_basis, cutoff_kind;
  float r_max, cutoff_r_min, cutoff_r_max, cutoff_p, cutoff_eps;
} eqt_edge_features;
int eqt_radius_count(const eqt_radius_grid* grid, const float* pos, const int64_t* batch, int64_t n, float r, int32_t loop,
                     int32_t max_neighbors, int32_t* degree, int32_t* status, void* stream);
int eqt_radius_edges(const eqt_radius_grid* grid, const float* pos, const int64_t* batch, int64_t n, float r, int32_t loop,
                     int32_t max_neighbors, const int64_t* ptr, int64_t* src, int64_t* dst, const eqt_edge_features* features,
                     int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* EQT_B200_H */
