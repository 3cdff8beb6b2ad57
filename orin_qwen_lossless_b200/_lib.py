"""ctypes binding of libbf16n_b200.so (the C ABI declared in include/bf16n_c.h).

The library is the only implementation: if it is missing it is built with nvcc, and if that fails the import fails.
There is no Python, PyTorch or CPU fallback for any operator.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

_PKG = os.path.dirname(os.path.abspath(__file__))

OK, EINVAL, ECUDA, EINTERNAL = 0, 1, 2, 3


class Weight(C.Structure):
    """struct bf16n_weight"""
    _fields_ = [("plane", C.c_void_p), ("aux", C.c_void_p), ("format", C.c_int32), ("R", C.c_int32), ("K", C.c_int64),
                ("rows", C.c_int64), ("cm", C.c_int32), ("fo", C.c_int32), ("off_a", C.c_uint64), ("off_b", C.c_uint64),
                ("off_c", C.c_uint64), ("off_d", C.c_uint64)]


class MmvArgs(C.Structure):
    """struct bf16n_mmv_args"""
    _fields_ = [("x", C.c_void_p), ("x_bf16", C.c_int32), ("y", C.c_void_p), ("y_bf16", C.c_int32), ("ncols", C.c_int32),
                ("n_used", C.c_int32), ("x_per_slot", C.c_int32), ("x_tok", C.c_int64), ("y_tok", C.c_int64),
                ("ids", C.c_void_p), ("ids_s0", C.c_int64), ("ids_s1", C.c_int64), ("x_slot", C.c_int64),
                ("y_slot", C.c_int64), ("rows_per_matrix", C.c_int64), ("row0", C.c_int64), ("nrows", C.c_int64)]


class EpLayout(C.Structure):
    """struct bf16n_ep_layout"""
    _fields_ = [("n_ranks", C.c_int), ("rank", C.c_int), ("cap", C.c_int), ("K", C.c_int), ("H", C.c_int), ("n_pairs_max", C.c_int),
                ("base", C.c_void_p * 8), ("off_counts", C.c_size_t), ("off_expert", C.c_size_t), ("off_pair", C.c_size_t),
                ("off_rows", C.c_size_t), ("off_back", C.c_size_t)]


class PeerOut(C.Structure):
    """struct bf16n_peer_out"""
    _fields_ = [("n_peers", C.c_int), ("y", C.c_void_p * 7), ("flag", C.c_void_p * 7), ("local_header", C.c_void_p), ("wait_mask", C.c_int)]


# name -> (restype, argtypes); every symbol include/bf16n_c.h declares
SIGNATURES = {
    "bf16n_last_error": (C.c_char_p, []),
    "bf16n_encode": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "bf16n_encoded_plane": (C.c_void_p, [C.c_void_p, C.POINTER(C.c_size_t)]),
    "bf16n_encoded_aux": (C.c_void_p, [C.c_void_p, C.POINTER(C.c_size_t)]),
    "bf16n_encoded_format": (C.c_int, [C.c_void_p]),
    "bf16n_encoded_R": (C.c_int, [C.c_void_p]),
    "bf16n_encoded_free": (None, [C.c_void_p]),
    "bf16n_parse_header": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(Weight)]),
    "bf16n_choose": (C.c_int, [C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int64, C.c_int, C.c_int, C.POINTER(C.c_int)]),
    "bf16n_choose_for_machine": (C.c_int, [C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int64,
                                           C.POINTER(C.c_int)]),
    "bf16n_init": (C.c_int, []),
    "bf16n_sm_count": (C.c_int, [C.POINTER(C.c_int)]),
    "bf16n_mmv": (C.c_int, [C.POINTER(Weight), C.POINTER(MmvArgs), C.c_void_p, C.c_int]),
    "bf16n_mmv_group": (C.c_int, [C.POINTER(Weight), C.POINTER(MmvArgs), C.c_int, C.c_void_p]),
    "bf16n_mmv_glu_merged": (C.c_int, [C.POINTER(Weight), C.POINTER(MmvArgs), C.c_void_p]),
    "bf16n_mmv_glu": (C.c_int, [C.POINTER(Weight), C.POINTER(Weight), C.POINTER(MmvArgs), C.c_void_p]),
    "bf16n_dequant": (C.c_int, [C.POINTER(Weight), C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "bf16n_verify": (C.c_int, [C.POINTER(Weight), C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "bf16n_get_rows": (C.c_int, [C.POINTER(Weight), C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int, C.c_int64, C.c_void_p, C.c_int64]),
    "bf16n_mm_ids_supported": (C.c_int, [C.POINTER(Weight), C.POINTER(Weight)]),
    "bf16n_mm_ids_workspace_bytes": (C.c_size_t, [C.POINTER(Weight), C.POINTER(Weight)]),
    "bf16n_set_workspace": (C.c_int, [C.c_void_p, C.c_size_t]),
    "bf16n_mm_ids_route": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "bf16n_mm_ids": (C.c_int, [C.POINTER(Weight), C.POINTER(Weight), C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "bf16n_moe_combine": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_void_p]),
    "bf16n_swiglu": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "bf16n_moe_decode_scratch_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int64, C.c_int64]),
    "bf16n_moe_decode": (C.c_int, [C.POINTER(Weight), C.POINTER(Weight), C.POINTER(Weight), C.c_void_p, C.c_int, C.c_int64, C.c_void_p,
                                   C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_size_t,
                                   C.c_void_p, C.c_int, C.c_void_p]),
    "bf16n_moe_decode_static": (C.c_int, [C.POINTER(Weight), C.POINTER(Weight), C.POINTER(Weight), C.c_void_p, C.c_int, C.c_int64,
                                          C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                          C.c_int, C.c_void_p]),
    "bf16n_moe_topk": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "bf16n_exchange_create": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p]),
    "bf16n_exchange_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "bf16n_exchange_close": (C.c_int, [C.c_void_p]),
    "bf16n_exchange_destroy": (C.c_int, [C.c_void_p]),
    "bf16n_mmv_peers": (C.c_int, [C.POINTER(Weight), C.POINTER(MmvArgs), C.POINTER(PeerOut), C.c_void_p]),
    "bf16n_moe_decode_peers": (C.c_int, [C.POINTER(Weight), C.POINTER(Weight), C.POINTER(Weight), C.c_void_p, C.c_int, C.c_int64, C.c_void_p,
                                         C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_size_t,
                                         C.c_void_p, C.c_int, C.POINTER(PeerOut), C.c_void_p]),
    "bf16n_peer_sum": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "bf16n_peer_wait": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "bf16n_peer_expired": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int)]),
    "bf16n_set_peer_wait_limit_ms": (C.c_int, [C.c_uint]),
    "bf16n_ep_layout_bytes": (C.c_size_t, [C.POINTER(EpLayout)]),
    "bf16n_ep_dispatch": (C.c_int, [C.POINTER(EpLayout), C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "bf16n_ep_inbox_ids": (C.c_int, [C.POINTER(EpLayout), C.c_void_p, C.c_void_p]),
    "bf16n_ep_give_back": (C.c_int, [C.POINTER(EpLayout), C.c_void_p, C.c_void_p]),
    "bf16n_adapter_choose": (C.c_int, [C.c_int64, C.c_int64, C.c_int64, C.c_char_p, C.c_int64, C.c_int]),
    "bf16n_adapter_convert": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_char_p,
                                        C.POINTER(C.c_int)]),
    "bf16n_adapter_lookup": (C.c_int, [C.c_void_p, C.POINTER(Weight), C.POINTER(C.c_int64)]),
    "bf16n_adapter_release": (C.c_int, [C.c_void_p]),
    "bf16n_adapter_count": (C.c_int, []),
    "bf16n_int4_quantize": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "bf16n_int2_quantize": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "bf16n_int4_gemv": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]),
    "bf16n_int2_gemv": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]),
    "bf16n_fault_status": (C.c_int, [C.POINTER(C.c_uint), C.c_void_p]),
}

_lib = None


def lib():
    """The loaded library (built first when the .so is absent or older than its sources and nvcc is available)."""
    global _lib
    if _lib is None:
        path = _build.LIB
        if not os.path.exists(path):
            _build.build()
        _lib = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(_lib, name)  # AttributeError here = the library does not export what the header declares
            fn.restype = res
            fn.argtypes = args
    return _lib


def check(rc: int) -> None:
    """Map a status code to the exception the reference raises: ValueError for invalid arguments, RuntimeError else."""
    if rc == OK:
        return
    msg = (lib().bf16n_last_error() or b"").decode()
    if rc == EINVAL:
        raise ValueError(msg)
    raise RuntimeError(msg)
