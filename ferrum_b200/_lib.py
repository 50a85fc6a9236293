"""ctypes binding of ``libferrum_b200.so`` (the C ABI declared in ``include/ferrum_b200.h``).

There is no fallback: if the shared library is missing or fails to load, importing the package's
compute surface raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libferrum_b200.so")

OK, ERR_SHAPE, ERR_RANGE, ERR_DEVICE, ERR_ALIAS, ERR_WEIGHT, ERR_SYNC, ERR_TIMEOUT, ERR_CUDA, ERR_PARAM, \
    ERR_UNSUPPORTED, ERR_GGUF = range(12)
Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS = 8, 12, 13, 14, 20, 23
F32, BF16 = 0, 30


class MatrixInfo(C.Structure):
    _fields_ = [("rows", C.c_uint64), ("cols", C.c_uint64), ("experts", C.c_uint64),
                ("row_bytes", C.c_uint64), ("byte_size", C.c_uint64), ("format", C.c_int32)]


class Counters(C.Structure):
    _fields_ = [("dispatches", C.c_uint64), ("synchronizes", C.c_uint64),
                ("bytes_uploaded", C.c_uint64), ("bytes_downloaded", C.c_uint64)]


class ProfileEntry(C.Structure):
    _fields_ = [("name", C.c_char * 48), ("calls", C.c_uint64), ("kernels", C.c_uint64), ("wall_ns", C.c_uint64),
                ("gpu_ns", C.c_uint64), ("gpu_samples", C.c_uint64)]


class GgufTensor(C.Structure):
    _fields_ = [("name", C.c_char * 260), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 4), ("type_id", C.c_uint32),
                ("offset", C.c_uint64), ("byte_len", C.c_uint64)]


class GgufInfo(C.Structure):
    _fields_ = [("version", C.c_uint32), ("alignment", C.c_uint32), ("file_len", C.c_uint64), ("tensor_data_offset", C.c_uint64),
                ("tensor_count", C.c_uint64), ("metadata_count", C.c_uint64)]


class MoeFfnDesc(C.Structure):
    _fields_ = [("router", C.c_void_p), ("gate_exps", C.c_void_p), ("up_exps", C.c_void_p),
                ("down_exps", C.c_void_p), ("shared_gate", C.c_void_p), ("shared_up", C.c_void_p),
                ("shared_down", C.c_void_p), ("shared_gate_inp", C.c_void_p),
                ("experts", C.c_uint32), ("used", C.c_uint32), ("hidden", C.c_uint32),
                ("expert_ffn", C.c_uint32), ("shared_ffn", C.c_uint32),
                ("sigmoid", C.c_int32), ("norm_weights", C.c_int32)]


# name -> (restype, argtypes); every symbol the header declares.
_P, _Z, _I, _U32, _U64 = C.c_void_p, C.c_size_t, C.c_int, C.c_uint32, C.c_uint64
SIGNATURES = {
    "fq_device_create": (_I, [_I, C.POINTER(_P)]),
    "fq_device_destroy": (_I, [_P]),
    "fq_device_set_stream": (_I, [_P, _P]),
    "fq_device_stream": (_P, [_P]),
    "fq_synchronize": (_I, [_P]),
    "fq_device_recover": (_I, [_P]),
    "fq_last_error": (C.c_char_p, [_P]),
    "fq_status_name": (C.c_char_p, [_I]),
    "fq_get_counters": (_I, [_P, C.POINTER(Counters)]),
    "fq_set_exact": (_I, [_P, _I]),
    "fq_test_fail_after": (_I, [_P, _I]),
    "fq_test_fail_completion": (_I, [_P]),
    "fq_probe_read_stream": (_I, [_P, _P, _Z, _U32]),
    "fq_set_profiling": (_I, [_P, _I]),
    "fq_take_profile": (_I, [_P, C.POINTER(ProfileEntry), _Z, C.POINTER(_Z)]),
    "fq_capture_begin": (_I, [_P]),
    "fq_capture_end": (_I, [_P, C.POINTER(_P)]),
    "fq_graph_launch": (_I, [_P, _P]),
    "fq_graph_destroy": (_I, [_P]),
    "fq_buffer_alloc": (_I, [_P, _Z, C.POINTER(_P)]),
    "fq_buffer_free": (_I, [_P, _P]),
    "fq_upload": (_I, [_P, _P, _P, _Z]),
    "fq_download": (_I, [_P, _P, _P, _Z]),
    "fq_download_async": (_I, [_P, _P, _P, _Z]),
    "fq_matrix_create": (_I, [_P, _I, _U64, _U64, _U64, _P, _Z, C.POINTER(_P)]),
    "fq_matrix_destroy": (_I, [_P]),
    "fq_matrix_get_info": (_I, [_P, C.POINTER(MatrixInfo)]),
    "fq_gguf_open": (_I, [C.c_char_p, _I, _U64, C.POINTER(_P), C.c_char_p, _Z]),
    "fq_gguf_close": (_I, [_P]),
    "fq_gguf_last_error": (C.c_char_p, [_P]),
    "fq_gguf_info": (_I, [_P, C.POINTER(GgufInfo)]),
    "fq_gguf_tensor_by_name": (_I, [_P, C.c_char_p, C.POINTER(GgufTensor)]),
    "fq_gguf_tensor_by_index": (_I, [_P, _U64, C.POINTER(GgufTensor)]),
    "fq_gguf_read_tensor": (_I, [_P, C.c_char_p, _P, _Z]),
    "fq_gguf_metadata_u64": (_I, [_P, C.c_char_p, C.POINTER(_U64)]),
    "fq_gguf_metadata_f64": (_I, [_P, C.c_char_p, C.POINTER(C.c_double)]),
    "fq_gguf_metadata_string": (_I, [_P, C.c_char_p, C.c_char_p, _Z]),
    "fq_gguf_metadata_array": (_I, [_P, C.c_char_p, C.POINTER(_U32), C.POINTER(_U64), C.POINTER(_U64)]),
    "fq_block_layout": (_I, [_U32, C.POINTER(_U32), C.POINTER(_U32)]),
    "fq_matrix_from_gguf": (_I, [_P, _P, C.c_char_p, _U64, _U64, _U64, _I, C.POINTER(_P)]),
    "fq_q3k_to_q6k": (_I, [_P, _Z, _P]),
    "fq_quantize_q8_0": (_I, [_P, _Z, _P]),
    "fq_project": (_I, [_P, _P, _P, _I, _Z, _Z, _P, _I, _Z]),
    "fq_project_many": (_I, [_P, C.POINTER(_P), _Z, _P, _I, _Z, _Z, C.POINTER(_P), _I]),
    "fq_rmsnorm": (_I, [_P, _P, _P, _U32, C.c_float, _U32, _P]),
    "fq_add_rmsnorm": (_I, [_P, _P, _P, _P, _U32, C.c_float, _U32, _P, _P]),
    "fq_rmsnorm_project_many": (_I, [_P, C.POINTER(_P), _Z, _P, _P, C.c_float, _Z, _Z, _P, C.POINTER(_P)]),
    "fq_argmax": (_I, [_P, _P, _U32, _U32, _P]),
    "fq_topk_blocks": (_I, [_P, _P, _U32, _U32, _P]),
    "fq_project_id": (_I, [_P, _P, _P, _Z, _P, _Z, _Z, _P, _Z]),
    "fq_project_mm_id": (_I, [_P, _P, _P, _I, _Z, _P, _P, _Z, _Z, _P, _I, _Z]),
    "fq_get_rows": (_I, [_P, _P, _P, _Z, _P, _I, _Z]),
    "fq_moe_route": (_I, [_P, _P, _P, _P, _U32, _U32, _U32, _U32, _I, _I, _I, _P, _P, _P]),
    "fq_moe_map": (_I, [_P, _P, _U32, _U32, _P, _P, _P]),
    "fq_moe_gather": (_I, [_P, _P, _P, _U32, _U32, _U32, _P]),
    "fq_moe_combine": (_I, [_P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _I, _P]),
    "fq_glu": (_I, [_P, _P, _P, _Z, _P]),
    "fq_dense_ffn": (_I, [_P, _P, _P, _P, _P, _Z, _P, _Z, _P]),
    "fq_moe_ffn_scratch_elems": (_Z, [C.POINTER(MoeFfnDesc), _Z]),
    "fq_moe_ffn": (_I, [_P, C.POINTER(MoeFfnDesc), _P, _Z, _P, _Z, _P]),
    "fq_project_host": (_I, [_P, _P, _P, _Z, _P]),
    "fq_comm_create": (_I, [_P, _I, _I, _Z, C.POINTER(_P)]),
    "fq_comm_handle": (_I, [_P, _P]),
    "fq_comm_open": (_I, [_P, _P]),
    "fq_comm_buffer": (_P, [_P]),
    "fq_comm_all_gather": (_I, [_P, _P, _Z, _Z]),
    "fq_comm_all_gather_rows": (_I, [_P, _P, _Z, _Z, _P, _U32, _Z]),
    "fq_comm_destroy": (_I, [_P]),
    "fq_comm_set_wait_ns": (_I, [_P, _U64]),
    "fq_comm_open_local": (_I, [_P]),
    "fq_project_many_gather": (_I, [_P, _P, _Z, _Z, C.POINTER(_P), _Z, _P, _I, _Z, _Z, C.POINTER(_P), _I]),
    "fq_moe_ffn_ep": (_I, [_P, _P, _Z, C.POINTER(MoeFfnDesc), _U32, _P, _Z, _P, _Z, _P]),
    "fq_gemv_q4k_static": (_I, [_P, _U64, _U64, _P, _U32, _P, _P, C.c_char_p, _Z]),
    "fq_project_many_host": (_I, [_P, C.POINTER(_P), _Z, _P, _Z, C.POINTER(_P)]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library and attach the prototypes.  Raises if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m ferrum_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError here means the library is stale
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib
