"""ctypes binding of libq4k_b200.so (the C ABI declared in include/q4k_b200.h).

The library is the product: if it is missing, importing this module builds it with nvcc,
and if that is impossible it raises.  There is no CPU or PyTorch fallback."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from . import build as _build

OK, ERR_STATUS, ERR_INVALID_ARGUMENT, ERR_OVERFLOW = 0, 1, 2, 3
LAYOUT_SPLIT_TILES, QUANTIZER_Q4K = 0x020D, 0x0105
KERNEL_AUTO, KERNEL_GEMV_DP4A, KERNEL_MMA, KERNEL_TCGEN05, KERNEL_GEMV_MMA, KERNEL_GEMV_TMA = 0, 1, 2, 3, 4, 5
FLAG_TRUSTED_SPANS = 1


class Weight(C.Structure):
    _fields_ = [("codes", C.c_void_p), ("scales", C.c_void_p), ("layout", C.c_uint16),
                ("quantizer", C.c_uint16), ("n", C.c_uint32), ("k", C.c_uint32),
                ("padded_n", C.c_uint32), ("padded_k", C.c_uint32),
                ("codes_bytes", C.c_uint64), ("scales_bytes", C.c_uint64)]


class Q8(C.Structure):
    _fields_ = [("codes", C.c_void_p), ("scales", C.c_void_p), ("sums", C.c_void_p),
                ("codes_len", C.c_uint64), ("scales_len", C.c_uint64), ("sums_len", C.c_uint64),
                ("m", C.c_uint32), ("k", C.c_uint32), ("padded_k", C.c_uint32)]


class ProjectOptions(C.Structure):
    _fields_ = [("kernel", C.c_uint32), ("split_k", C.c_uint32), ("row_groups", C.c_uint32), ("partials", C.c_void_p),
                ("partials_len", C.c_uint64), ("workspace", C.c_void_p),
                ("workspace_bytes", C.c_uint64), ("flags", C.c_uint32)]


class DecodeDesc(C.Structure):
    _fields_ = [("weight", Weight), ("input", C.c_void_p), ("input_len", C.c_uint64), ("output", C.c_void_p),
                ("output_len", C.c_uint64), ("residual", C.c_void_p), ("residual_len", C.c_uint64), ("m", C.c_uint32),
                ("epilogue", C.c_uint8), ("activation_policy", C.c_uint8)]


FLAG_TRUSTED_SPANS, FLAG_INPUT_SETTLED = 1, 2
EPILOGUE_STORE_BF16, EPILOGUE_STORE_FP32, EPILOGUE_RESIDUAL_ADD_FP32, EPILOGUE_SWIGLU_STORE_BF16 = 1, 2, 3, 4
ACTIVATION_BF16, ACTIVATION_Q8_K32 = 1, 2


class GatherDesc(C.Structure):
    _fields_ = [("outputs", C.c_void_p * 8), ("flags", C.c_void_p * 8), ("ranks", C.c_uint32), ("rank", C.c_uint32),
                ("row_offset", C.c_uint32), ("total_rows", C.c_uint32), ("options", C.c_uint32)]


_u32, _u64, _vp, _i = C.c_uint32, C.c_uint64, C.c_void_p, C.c_int
_WP, _OP = C.POINTER(Weight), C.POINTER(ProjectOptions)

# name -> (restype, argtypes); kept in step with include/q4k_b200.h by tests/test_abi.py.
SIGNATURES = {
    "q4k_last_error": (C.c_char_p, []),
    "q4k_last_cuda_status": (_i, []),
    "q4k_abi_version": (_u32, []),
    "q4k_kernel_status": (_i, [C.POINTER(_i)]),
    "q4k_reserve_scratch": (_i, [_u64, _vp]),
    "q4k_measure_int8_peak": (_i, [_u32, C.POINTER(C.c_double), C.POINTER(C.c_double), _vp]),
    "q4k_set_profiling_ranges": (None, [_i]),
    "q4k_get_profiling_ranges": (_i, []),
    "q4k_session_create": (_i, [_u64, C.POINTER(_vp)]),
    "q4k_session_destroy": (None, [_vp]),
    "q4k_session_workspace": (_vp, [_vp]),
    "q4k_session_workspace_bytes": (_u64, [_vp]),
    "q4k_session_failure": (_vp, [_vp]),
    "q4k_session_take_failure": (_i, [_vp, _vp]),
    "q4k_set_launch_overlap": (None, [_i]),
    "q4k_get_launch_overlap": (_i, []),
    "q4k_pad_n": (_u64, [_u32]),
    "q4k_pad_k": (_u32, [_u32]),
    "q4k_code_bytes": (_u64, [_u32, _u32]),
    "q4k_scale_bytes": (_u64, [_u32, _u32]),
    "q4k_validate_device_span": (_i, [_vp, _u64, _u32, _i]),
    "q4k_pack_q8_bf16": (_i, [_vp, _u64, Q8, _vp, _vp]),
    "q4k_pack_q8_f32": (_i, [_vp, _u64, Q8, _vp, _vp]),
    "q4k_export_q8_1": (_i, [Q8, _vp, _u64, _vp]),
    "q4k_q8_project": (_i, [_WP, Q8, _vp, _u64, _vp, _u64, _vp]),
    "q4k_q8_project_ex": (_i, [_WP, Q8, _vp, _u64, _vp, _u64, _OP, _vp]),
    "q4k_q8_project_static": (_i, [_WP, Q8, _vp, _u64, _vp, _u64, _u32, _vp]),
    "q4k_project_workspace_bytes": (_u64, [_u32, _u32, _u32]),
    "q4k_decode_workspace_bytes": (_u64, [_u32, _u64, _u32]),
    "q4k_decode_mmv": (_i, [C.POINTER(DecodeDesc), _vp, _u64, _vp, _vp]),
    "q4k_decode_mmv_paired": (_i, [C.POINTER(DecodeDesc), C.POINTER(DecodeDesc), _vp, _u64, _vp, _vp]),
    "q4k_decode_mmv_ranges": (_i, [C.POINTER(DecodeDesc), _u32, _vp, _u64, _vp, _vp]),
    "q4k_prefill_project": (_i, [C.POINTER(DecodeDesc), _vp, _u64, _vp, _vp]),
    "q4k_prefill_paired_swiglu": (_i, [_WP, _WP, _vp, _vp, _u32, _vp, _u64, _vp, _vp]),
    "q4k_q8_project_gather": (_i, [_WP, Q8, C.POINTER(GatherDesc), _vp, _u64, _vp]),
    "q4k_peer_wait": (_i, [C.POINTER(GatherDesc), _u64, _vp]),
    "q4k_peer_announce": (_i, [C.POINTER(GatherDesc), _vp]),
    "q4k_q8_project_ragged": (_i, [_WP, Q8, C.POINTER(_u32), _u32, _vp, _u64, _OP, _vp]),
    "q4k_repack_blocks144": (_i, [_vp, _u64, _u32, _u32, _vp, _u64, _vp, _u64, _vp]),
    "q4k_validate_weight": (_i, [_WP, _vp, _vp]),
    "q4k_dequantize_bf16": (_i, [_WP, _vp, _u64, _vp]),
    "q4k_unpack_logical": (_i, [_WP, _vp, _u64, _vp, _u64, _vp]),
    "q4k_fit_blocks": (_i, [_vp, _u32, _u64, _vp, _vp, _vp, _vp, _vp]),
    "q4k_fit_weight": (_i, [_vp, _u32, _u32, _u32, _vp, _u64, _vp, _u64, _vp, _vp, _vp]),
    "q4k_q8_mlp_workspace_bytes": (_u64, [_u32, _u32, _u32]),
    "q4k_q8_mlp": (_i, [_WP, _WP, _WP, _vp, _vp, C.c_float, _vp, _u32, _vp, _u64, _vp,
                        C.POINTER(_i), _vp]),
    "q4k_hidden_rms_q8": (_i, [_vp, _vp, C.c_float, _u32, _u32, Q8, _vp, _vp]),
    "q4k_swiglu_pack_q8": (_i, [_vp, _vp, _u32, _u32, Q8, _vp, _vp]),
}

_lib = None


def library_path() -> Path:
    return _build.LIB


def load() -> C.CDLL:
    """Load (building first if the sources are newer) and type every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    import os
    override = os.environ.get("Q4K_B200_LIBRARY")  # an already-built library to load instead
    path = override if override else _build.build()
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library disagree
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib
