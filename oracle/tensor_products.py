"""ORACLE (test infrastructure, never imported by the product path).

Two CPU restatements of the reference's tensor-product layers, both plain
differentiable PyTorch so autograd yields the gradients the reference writes out by
hand (equitorch/nn/functional/linears.py:16-492, tensor_products.py:9-172):

1. **dense path form** (`so3_linear_dense`, `tensor_product_dense`): one einsum per
   coupling path ``(k, i, j)`` with the dense real CG block, normalised like
   ``prepare_so3`` (equitorch/utils/_structs.py:162-216).  It never touches the sparse
   index tables, so it checks table construction and kernels together.
2. **sparse composition form** (`so3_linear_sparse`, ...): the same two-step chains the
   reference runs (CG contraction -> weight step) on the restated sparse ops of
   ``oracle.sparse_ops`` with the ``TensorProductInfo`` tables.

The message-passing form adds what surrounds the layer in a graph network: gather node
features by edge source, spherical harmonics of the edge vector, the layer, and a sum
over edges into their destination node.  The reference has no code for the gather and
the reduction (users call a third-party scatter), so that part is defined here as a
plain ``index_select`` / ``index_add`` and is **parity unpinned** against the reference.

Pinned against reference outputs in tests/golden.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
from torch import Tensor

from equitorch_b200.constants import so3_clebsch_gordan
from equitorch_b200.irreps import Irreps, check_irreps, has_path, irrep_segments

from . import sparse_ops as ops
from .sphericals import spherical_harmonics


def _paths(irreps_out: Irreps, irreps1: Irreps, irreps2: Irreps, path=None):
    if not path:
        path = [(k, i, j) for k, a in enumerate(irreps_out) for i, b in enumerate(irreps1)
                for j, c in enumerate(irreps2) if has_path(a, b, c)]
    fan, prev = {}, None
    for k, _, _ in path:
        fan[k] = fan[k] + 1 if k == prev else 1
        prev = k
    return path, fan


def _blocks(irreps: Irreps):
    seg = irrep_segments(irreps)
    return [(seg[n], seg[n + 1]) for n in range(len(seg) - 1)]


def _tp_dense(mode: str, x: Tensor, y: Tensor, weight: Tensor, irreps_in1, irreps_in2, irreps_out,
              path=None, path_norm=True, channel_norm=False, channel_scale=1.0) -> Tensor:
    ir1, ir2, iro = check_irreps(irreps_in1), check_irreps(irreps_in2), check_irreps(irreps_out)
    path, fan = _paths(iro, ir1, ir2, path)
    b1, b2, bo = _blocks(ir1), _blocks(ir2), _blocks(iro)
    l1, l2, lo = [ir.l for ir in ir1], [ir.l for ir in ir2], [ir.l for ir in iro]
    shared = weight.dim() == {"uu": 2, "uv": 3, "uuu": 2, "uvw": 4}[mode]
    n = x.shape[0]
    c_out = x.shape[-1] if mode in ("uu", "uuu") else weight.shape[-1]
    out = [x.new_zeros(n, hi - lo_, c_out) for lo_, hi in bo]
    eq = {"uu": ("mab,nac,nb,c->nmc", "mab,nac,nb,nc->nmc"),
          "uv": ("mab,nac,nb,cd->nmd", "mab,nac,nb,ncd->nmd"),
          "uuu": ("mab,nac,nbc,c->nmc", "mab,nac,nbc,nc->nmc"),
          "uvw": ("mab,nac,nbd,cde->nme", "mab,nac,nbd,ncde->nme")}[mode][0 if shared else 1]
    for w, (k, i, j) in enumerate(path):
        norm = (fan[k] ** (-0.5) if path_norm else 1.0) * (channel_scale if channel_norm else 1.0)
        cg = torch.as_tensor(so3_clebsch_gordan(lo[k], l1[i], l2[j]) * norm, dtype=x.dtype, device=x.device)
        xi = x[:, b1[i][0]:b1[i][1]]
        yj = y[:, b2[j][0]:b2[j][1]]
        wp = weight[w] if shared else weight[:, w]
        out[k] = out[k] + torch.einsum(eq, cg, xi, yj, wp)
    return torch.cat(out, dim=1)


def so3_linear_dense(x, y, weight, irreps_in1, irreps_in2, irreps_out, feature_mode="uu", **kw):
    """SO3Linear: ``y`` has no channel axis (equitorch/nn/linears.py:26-212)."""
    return _tp_dense(feature_mode, x, y, weight, irreps_in1, irreps_in2, irreps_out, **kw)


def tensor_product_dense(x, y, weight, irreps_in1, irreps_in2, irreps_out, feature_mode="uuu", **kw):
    """TensorProduct: both operands carry channels (equitorch/nn/tensor_products.py:19-198)."""
    return _tp_dense(feature_mode, x, y, weight, irreps_in1, irreps_in2, irreps_out, **kw)


# ---- sparse composition form -------------------------------------------------------
def _call(fn, a, b, info):
    return fn(a, b, info.scale, info.index1, info.index2, info.seg_out, info.gather_index,
              info.index_out, out_size=info.out_size)


def so3_linear_sparse(x, y, weight, tp_info, feature_mode="uu"):
    inter = _call(ops.indexed_vecsca_scale_gather, x, y, tp_info.info_Mij_fwd)
    step = ops.indexed_mul_scale_gather if feature_mode == "uu" else ops.indexed_vecmat_scale_gather
    return _call(step, inter, weight, tp_info.info_M_fwd)


def tensor_product_sparse(x, y, weight, tp_info, feature_mode="uuu"):
    if feature_mode == "uuu":
        inter = _call(ops.indexed_mul_scale_gather, x, y, tp_info.info_Mij_fwd)
        return _call(ops.indexed_mul_scale_gather, inter, weight, tp_info.info_M_fwd)
    inter = _call(ops.indexed_outer_scale_gather, x, y, tp_info.info_Mij_fwd)
    return _call(ops.indexed_vecmat_scale_gather, inter.flatten(-2), weight.flatten(-3, -2), tp_info.info_M_fwd)


def so2_linear_sparse(x, weight, info, feature_mode="uu"):
    step = ops.indexed_mul_scale_gather if feature_mode == "uu" else ops.indexed_vecmat_scale_gather
    return _call(step, x, weight, info)


def irrep_wise_linear(x, weight, irrep_index):
    """``out[n, M, :] = x[n, M, :] @ W[irrep(M)]`` (equitorch/nn/functional/linears.py:494-530)."""
    w = weight.index_select(-3, irrep_index)
    return torch.einsum("nmi,...mio->nmo", x, w)


def sparse_wigner_rotation(x, cs_alpha, cs_beta, cs_gamma, info):
    """``Dz(alpha) J Dz(beta) J Dz(gamma) x`` on the sparse ops
    (equitorch/nn/functional/wigner_d.py:14-56)."""
    z, j = info.rotate_z_info_fwd, info.j_matrix_info
    if cs_gamma is not None:
        x = _call(ops.indexed_vecsca_scale_gather, x, cs_gamma, z)
    if cs_beta is not None:
        x = ops.indexed_scale_segment(x, j.scale, j.index, j.seg_out, j.out_size)
        x = _call(ops.indexed_vecsca_scale_gather, x, cs_beta, z)
        x = ops.indexed_scale_segment(x, j.scale, j.index, j.seg_out, j.out_size)
    if cs_alpha is not None:
        x = _call(ops.indexed_vecsca_scale_gather, x, cs_alpha, z)
    return x


# ---- message passing (gather -> SH -> layer -> sum into destination nodes) ----------
def so3_linear_message_passing(node_x: Tensor, edge_vec: Tensor, src: Tensor, dst: Tensor,
                               weight: Tensor, irreps_in1, irreps_in2, irreps_out,
                               feature_mode="uv", num_out_nodes: Optional[int] = None,
                               normalize: bool = True, **kw) -> Tensor:
    ir2 = check_irreps(irreps_in2)
    l_max = ir2.l_max
    v = torch.nn.functional.normalize(edge_vec, dim=-1) if normalize else edge_vec
    y = spherical_harmonics(v, l_max)
    msg = so3_linear_dense(node_x.index_select(0, src), y, weight, irreps_in1, ir2, irreps_out,
                           feature_mode=feature_mode, **kw)
    n_out = node_x.shape[0] if num_out_nodes is None else num_out_nodes
    return msg.new_zeros(n_out, *msg.shape[1:]).index_add(0, dst, msg)


def tensor_dot_uu(x1: Tensor, x2: Tensor, irreps, scaled: bool = True) -> Tensor:
    """Irrep-wise dot product of two channelled features, (N, D, C) x (N, D, C) -> (N, num_irreps, C); with
    ``scaled`` each irrep's sum is divided by sqrt(2l + 1) (equitorch/nn/functional/tensor_products.py:173-223,
    module equitorch/nn/tensor_products.py:199-269)."""
    ir = check_irreps(irreps)
    outs = []
    for (lo, hi) in _blocks(ir):
        d = (x1[:, lo:hi] * x2[:, lo:hi]).sum(dim=1)
        outs.append(d / (hi - lo) ** 0.5 if scaled else d)
    return torch.stack(outs, dim=1)
