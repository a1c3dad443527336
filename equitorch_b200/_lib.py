"""ctypes binding of ``libeqt_b200.so`` (the C ABI declared in ``include/eqt_b200.h``).

There is no fallback: if the shared library is missing or a kernel call fails, an
exception is raised.  Build the library with ``python -m equitorch_b200.csrc.build``.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libeqt_b200.so")

EQT_F32, EQT_F64, EQT_BF16 = 0, 1, 2
OP_MUL, OP_VECSCA, OP_SCALE, OP_OUTER, OP_INNER, OP_VECMAT = range(6)

DTYPE_CODE = {torch.float32: EQT_F32, torch.float64: EQT_F64, torch.bfloat16: EQT_BF16}


class EqtError(RuntimeError):
    pass


class ProductArgs(C.Structure):
    _fields_ = [
        ("op", C.c_int32), ("dtype", C.c_int32), ("shared1", C.c_int32), ("shared2", C.c_int32),
        ("accumulated", C.c_int32), ("reserved", C.c_int32),
        ("in1", C.c_void_p), ("in2", C.c_void_p), ("out", C.c_void_p), ("scale", C.c_void_p),
        ("index1", C.c_void_p), ("index2", C.c_void_p), ("seg", C.c_void_p),
        ("gather_index", C.c_void_p), ("index_out", C.c_void_p),
        ("n", C.c_int64), ("rows1", C.c_int64), ("rows2", C.c_int64), ("num_out", C.c_int64),
        ("out_size", C.c_int64), ("c1", C.c_int64), ("c2", C.c_int64),
    ]


class ShTable(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("m_out", C.c_void_p), ("m_in", C.c_void_p), ("axis", C.c_void_p),
                ("coef", C.c_void_p), ("l_max", C.c_int32), ("num_entries", C.c_int32)]


class TpTableStruct(C.Structure):
    _fields_ = [("scale", C.c_void_p), ("m_feat", C.c_void_p), ("m_y", C.c_void_p), ("row_ptr", C.c_void_p),
                ("num_entries", C.c_int32), ("num_rows", C.c_int32), ("d_feat", C.c_int32), ("d_y", C.c_int32),
                ("structure_key", C.c_uint64), ("scale_o", C.c_void_p)]


class WignerTableStruct(C.Structure):
    _fields_ = [("coef", C.c_void_p), ("comp", C.c_void_p), ("blocks", C.c_void_p), ("dim", C.c_int32),
                ("num_blocks", C.c_int32), ("max_l", C.c_int32), ("coef_count", C.c_int32)]


class RadiusGridStruct(C.Structure):
    _fields_ = [("cell_start", C.c_void_p), ("sorted_index", C.c_void_p), ("point_cell", C.c_void_p), ("cell_size", C.c_float),
                ("dims", C.c_int32 * 3)]


class EdgeFeaturesStruct(C.Structure):
    _fields_ = [("vec", C.c_void_p), ("length", C.c_void_p), ("sh", C.c_void_p), ("bessel", C.c_void_p), ("cutoff", C.c_void_p),
                ("bessel_weights", C.c_void_p), ("l_max", C.c_int32), ("integral_normalize", C.c_int32), ("num_basis", C.c_int32),
                ("cutoff_kind", C.c_int32), ("r_max", C.c_float), ("cutoff_r_min", C.c_float), ("cutoff_r_max", C.c_float),
                ("cutoff_p", C.c_float), ("cutoff_eps", C.c_float)]


class MixBlockStruct(C.Structure):
    _fields_ = [("in_row0", C.c_int32), ("out_row0", C.c_int32), ("dim", C.c_int32), ("paths", C.c_int32),
                ("w_offset", C.c_int64)]


# name -> (restype, argtypes); every symbol declared in include/eqt_b200.h appears here
SIGNATURES = {
    "eqt_sparse_product": (C.c_int, [C.POINTER(ProductArgs), C.c_void_p]),
    "eqt_sh_forward": (C.c_int, [C.c_int32, C.c_void_p, C.c_void_p, C.c_int64, C.POINTER(ShTable),
                                 C.c_int32, C.c_double, C.c_void_p]),
    "eqt_sh_backward": (C.c_int, [C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.POINTER(ShTable),
                                  C.c_int32, C.c_double, C.c_void_p]),
    "eqt_segment_sum": (C.c_int, [C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                  C.c_int64, C.c_void_p]),
    "eqt_gather_rows": (C.c_int, [C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "eqt_tp_cg_segment_sum": (C.c_int, [C.POINTER(TpTableStruct), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p]),
    "eqt_tp_cg_inner": (C.c_int, [C.POINTER(TpTableStruct), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                  C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p]),
    "eqt_mix_tc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32,
                             C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "eqt_mix_tc_transposed": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32,
                                        C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "eqt_wgrad_tc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_int32,
                               C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "eqt_wgrad_tc_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32,
                                      C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "eqt_wgrad_tc_static_capacity": (C.c_int64, []),
    "eqt_wgrad_tc_scratch_floats": (C.c_int64, [C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_int32]),
    "eqt_wigner_d_forward": (C.c_int, [C.POINTER(WignerTableStruct), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                       C.c_int32, C.c_void_p]),
    "eqt_wigner_d_backward": (C.c_int, [C.POINTER(WignerTableStruct), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p]),
    "eqt_dense_rotation": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                     C.c_int32, C.c_void_p]),
    "eqt_dense_rotation_grad_matrix": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p,
                                                 C.c_int32, C.c_void_p]),
    "eqt_vecmat_tc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p,
                                C.c_void_p]),
    "eqt_outer_tc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_int32,
                               C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                               C.c_int32, C.c_void_p, C.c_void_p]),
    "eqt_outer_tc_scratch_floats": (C.c_int64, [C.c_int64, C.c_int32, C.c_int32]),
    "eqt_radius_count": (C.c_int, [C.POINTER(RadiusGridStruct), C.c_void_p, C.c_void_p, C.c_int64, C.c_float, C.c_int32, C.c_int32,
                                   C.c_void_p, C.c_void_p, C.c_void_p]),
    "eqt_radius_edges": (C.c_int, [C.POINTER(RadiusGridStruct), C.c_void_p, C.c_void_p, C.c_int64, C.c_float, C.c_int32, C.c_int32,
                                   C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(EdgeFeaturesStruct), C.c_void_p, C.c_void_p]),
    "eqt_pack_weights": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_int32,
                                   C.c_void_p, C.c_void_p, C.c_void_p]),
    "eqt_irrep_scale": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32,
                                  C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "eqt_irrep_dot": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32,
                                C.c_int32, C.c_int32, C.c_void_p]),
    "eqt_layer_rms_num_partials": (C.c_int, [C.c_int64]),
    "eqt_layer_rms_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                                        C.c_int32, C.c_int32, C.c_int32, C.c_double, C.c_int32, C.c_void_p]),
    "eqt_layer_rms_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "eqt_last_error": (C.c_char_p, []),
    "eqt_version": (C.c_int, []),
    "eqt_launch_count": (C.c_int64, []),
}

_lock = threading.Lock()
_lib: Optional[C.CDLL] = None


def lib() -> C.CDLL:
    """Load (once) and return the shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise EqtError(
                        f"{LIB_PATH} is missing: the CUDA extension has not been built "
                        "(python -m equitorch_b200.csrc.build). There is no CPU fallback.")
                handle = C.CDLL(LIB_PATH)
                for name, (res, args) in SIGNATURES.items():
                    fn = getattr(handle, name)
                    fn.restype, fn.argtypes = res, args
                _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().eqt_last_error()
        raise EqtError(f"{what} failed with status {rc}: {msg.decode() if msg else ''}")


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    """All tensors must live on one CUDA device; returns it."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise EqtError("equitorch_b200 kernels run on CUDA tensors only (no CPU path): "
                           f"got a tensor on {t.device}")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise EqtError(f"tensors on different devices: {dev} and {t.device}")
    if dev is None:
        raise EqtError("no tensor given")
    return dev


def launch_count() -> int:
    return int(lib().eqt_launch_count())
