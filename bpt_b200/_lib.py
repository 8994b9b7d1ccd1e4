"""Loader of libbpt_b200.so, the C-ABI CUDA library declared in include/bpt_b200.h.

There is no CPU fallback: if the library has not been built, or no CUDA device is present
when a kernel is requested, the call raises.
"""
import ctypes
import os

import torch

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libbpt_b200.so")

F32, F64, BF16, F16 = 0, 1, 2, 3
_DTYPE_CODE = {torch.float32: F32, torch.float64: F64, torch.bfloat16: BF16, torch.float16: F16}

_i64, _int, _vp, _sz, _dbl = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_double

# name -> (restype, argtypes); mirrors include/bpt_b200.h declaration by declaration.
SIGNATURES = {
    "bpt_last_error": (ctypes.c_char_p, []),
    "bpt_version": (_int, []),
    "bpt_bp_levels": (_int, [_i64, _vp, _vp, _vp, _vp]),
    "bpt_bp_count_workspace_bytes": (_sz, [_i64]),
    "bpt_bp_count": (_int, [_i64, _int, _int, _int, _vp, _vp, _sz, _vp, _vp]),
    "bpt_bp_fill": (_int, [_i64, _int, _int, _int, _vp, _i64, _int, _vp, _vp, _vp, _vp, _vp]),
    "bpt_fc_count": (_int, [_i64, _int, _i64, _vp, _vp, _sz, _vp, _vp]),
    "bpt_fc_fill": (_int, [_i64, _int, _i64, _vp, _i64, _int, _vp, _vp, _vp, _vp, _vp]),
    "bpt_oas_count": (_int, [_i64, _i64, _i64, _vp, _vp, _sz, _vp, _vp]),
    "bpt_oas_fill": (_int, [_i64, _i64, _i64, _vp, _i64, _int, _vp, _vp, _vp, _vp, _vp]),
    "bpt_coo_to_csr_workspace_bytes": (_sz, [_i64, _i64]),
    "bpt_coo_to_csr": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _sz, _vp]),
    "bpt_partition_csr_workspace_bytes": (_sz, [_i64]),
    "bpt_partition_csr_count": (_int, [_vp, _i64, _int, _vp, _vp, _sz, _vp, _vp]),
    "bpt_partition_csr_fill": (_int, [_vp, _i64, _int, _vp, _i64, _vp, _vp, _vp]),
    "bpt_maskedmm_csr_forward": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _int, _int, _int, _vp]),
    "bpt_maskedmm_csr_backward": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64,
                                         _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _int, _vp]),
    "bpt_node_mul_edge_forward": (_int, [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _int, _int, _int, _vp]),
    "bpt_node_mul_edge_backward": (_int, [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _i64,
                                          _int, _int, _int, _vp]),
    "bpt_sparse_softmax_forward": (_int, [_vp, _vp, _vp, _i64, _vp, _vp, _int, _int, _vp]),
    "bpt_sparse_softmax_backward": (_int, [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _int, _int, _vp]),
    "bpt_vector_spmm_forward": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _int, _int, _int, _vp]),
    "bpt_vector_spmm_backward": (_int, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64,
                                        _vp, _vp, _vp, _vp, _vp, _i64, _int, _int, _int, _vp]),
    "bpt_attn_plan_bytes": (_sz, [_i64, _i64, _i64, _int]),
    "bpt_attn_plan_workspace_bytes": (_sz, [_i64, _i64, _i64, _int]),
    "bpt_attn_plan_build": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _sz, _vp, _sz, _vp, _vp]),
    "bpt_attn_workspace_bytes": (_sz, [_i64, _i64, _vp, _int, _int, _int]),
    "bpt_attn_forward": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _dbl, _vp, _vp,
                                _int, _int, _int, _vp, _sz, _vp, _vp]),
    "bpt_attn_backward": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _dbl, _vp, _vp,
                                 _vp, _vp, _vp, _vp, _int, _int, _int, _vp, _sz, _vp, _vp]),
    "bpt_attn_dropout_mask": (_int, [_vp, _vp, _i64, _int, _vp, _vp, _vp]),
    "bpt_tile_plan_create": (_vp, [_vp, _vp, _vp, _vp, _i64, _i64, _dbl, _int, _int, _int, _int, _int, _int]),
    "bpt_tile_plan_sizes": (_int, [_vp, _vp]),
    "bpt_tile_plan_export": (_int, [_vp, _vp, _vp, _vp, _vp, _int, _vp, _vp, _vp]),
    "bpt_tile_plan_destroy": (None, [_vp]),
    "bpt_tile_plan_create_device": (_vp, [_vp, _vp, _i64, _i64, _int, _int, _dbl, _int, _int, _int, _int, _vp]),
    "bpt_tile_plan_create_device_aligned": (_vp, [_vp, _vp, _i64, _i64, _int, _int, _vp, _int, _dbl, _int, _int, _int,
                                                  _int, _vp]),
    "bpt_tile_plan_device_sizes": (_int, [_vp, _vp]),
    "bpt_tile_plan_device_export": (_int, [_vp, _vp, _vp, _vp, _vp, _int, _vp, _vp, _vp]),
    "bpt_tile_plan_device_destroy": (None, [_vp]),
    "bpt_add_layer_norm": (_int, [_vp, _vp, _vp, _vp, _dbl, _vp, _i64, _int, _int, _vp]),
    "bpt_dense_blocks_fill": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _vp, _vp]),
    "bpt_export_in_csr": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _vp]),
    "bpt_export_out_csr": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _vp]),
    "bpt_attn_tc_smem_bytes": (_sz, [_int, _int, _int]),
    "bpt_attn_forward_tc32_smem_bytes": (_sz, [_int, _int, _int]),
    "bpt_attn_forward_tc32": (_int, [_vp, _i64, _int, _vp, _vp, _vp, _vp, _dbl, _vp, _vp, _int, _int, _vp, _sz, _vp, _vp]),
    "bpt_attn_backward_tc32_workspace_bytes": (_sz, [_vp, _vp, _vp, _i64, _i64, _int]),
    "bpt_attn_backward_tc32": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _dbl, _vp, _vp, _vp, _vp,
                                      _vp, _vp, _vp, _int, _int, _vp, _sz, _vp, _vp]),
    "bpt_attn_forward_tc_workspace_bytes": (_sz, [_i64, _int]),
    "bpt_attn_forward_tc": (_int, [_vp, _i64, _vp, _vp, _vp, _int, _vp, _i64, _i64, _vp, _i64, _vp, _vp,
                                   _i64, _i64, _int, _int, _int, _int, _int, _vp, _vp, _vp, _vp, _dbl, _vp,
                                   _vp, _int, _int, _int, _vp, _sz, _vp, _vp]),
    "bpt_attn_backward_tc_workspace_bytes": (_sz, [_vp, _vp, _vp, _i64, _i64, _int]),
    "bpt_attn_backward_tc": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _dbl, _vp, _vp, _vp,
                                    _vp, _vp, _vp, _vp, _int, _int, _int, _vp, _sz, _vp, _vp]),
    "bpt_attn_forward_tc5_smem_bytes": (_sz, [_int, _int]),
    "bpt_attn_forward_tc5_workspace_bytes": (_sz, [_i64, _int]),
    "bpt_attn_forward_tc5": (_int, [_vp, _i64, _int, _vp, _vp, _vp, _vp, _dbl, _vp, _vp, _int, _int, _int, _vp, _sz, _vp]),
    "bpt_attn_forward_tc5_status": (_int, [_vp, _vp, _vp]),
    "bpt_attn_forward_static": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _dbl, _vp, _vp,
                                       _int, _int, _int, _vp]),
}

class DropoutStruct(ctypes.Structure):
    """bpt_dropout_t of include/bpt_b200.h."""
    _fields_ = [("rate", ctypes.c_double), ("seed", ctypes.c_uint64)]


def dropout_arg(dropout):
    """dropout: None or (rate, seed).  Returns (keep-alive object, pointer value or None) for a bpt_dropout_t*."""
    if dropout is None or dropout[0] == 0:
        return None, None
    rate, seed = float(dropout[0]), int(dropout[1]) & 0xFFFFFFFFFFFFFFFF
    if not 0.0 <= rate < 1.0:
        raise RuntimeError("bpt_b200: dropout rate must be in [0, 1)")
    s = DropoutStruct(rate, seed)
    return s, ctypes.addressof(s)


class TilePlanStruct(ctypes.Structure):
    """bpt_tile_plan_t of include/bpt_b200.h."""
    _fields_ = [("groups", _vp), ("mblocks", _vp), ("cols", _vp), ("et", _vp), ("cell_pos", _vp),
                ("split_rows", _vp), ("row_items", _vp),
                ("n_groups", _i64), ("n_split", _i64), ("n_slots", _i64), ("n_row_items", _i64),
                ("et_bytes", ctypes.c_int32), ("max_cols_pad", ctypes.c_int32), ("t_max", ctypes.c_int32),
                ("reserved", ctypes.c_int32)]


_lib = None


def lib():
    """The loaded library. Raises if it was never built (python -m bpt_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "bpt_b200: %s is missing; build it with `python -m bpt_b200.build` "
                "(nvcc, sm_100a). There is no CPU fallback." % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc):
    if rc != 0:
        msg = lib().bpt_last_error()
        raise RuntimeError("bpt_b200 error %d: %s" % (rc, msg.decode() if msg else "unknown"))


def require_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("bpt_b200: expected a CUDA tensor (there is no CPU path)")
        if not t.is_contiguous():
            raise RuntimeError("bpt_b200: expected a contiguous tensor")


def ptr(t):
    return None if t is None else t.data_ptr()


def stream():
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dtype):
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise RuntimeError("bpt_b200: unsupported dtype %s" % dtype)


def workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=device)
