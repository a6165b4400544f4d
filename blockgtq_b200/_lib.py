"""ctypes binding of ``libbgtq.so`` (the C ABI declared in ``include/bgtq.h``).

There is no fallback: if the library is missing it is built in-tree with nvcc,
and if that is impossible importing an operator raises.  Tensors cross the
boundary as raw device pointers plus strides; torch is only the allocator and
stream provider.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import build as _build

HD = 128
MAX_SEG = 8
N_BINS = 256

OK = 0
ENC_K_NORMS_F16, ENC_K_MIXED, ENC_V_NIBBLE, ENC_SKIP_K, ENC_SKIP_V, ENC_FORCE_SIMT, ENC_PROGRAMMATIC = 1, 2, 4, 8, 16, 32, 64
ENC_NO_TCGEN05 = 128
DEC_K_MIXED, DEC_V_NIBBLE, DEC_PROGRAMMATIC, DEC_GENERIC = 1, 2, 4, 8
PF_NO_TCGEN05 = 16
COMBINE_PROGRAMMATIC = 1


class HeadDesc(C.Structure):
    """Mirror of ``BgtqHeadDesc``; field order and sizes must match the header."""
    _fields_ = [
        ("n_seg", C.c_int32), ("k_row_bytes", C.c_int32), ("v_bits", C.c_int32), ("v_row_bytes", C.c_int32),
        ("nopack_start", C.c_int32), ("nopack_len", C.c_int32), ("k_mixed_bytes", C.c_int32),
        ("reserved0", C.c_int32),
        ("seg_bw", C.c_int32 * MAX_SEG), ("seg_start", C.c_int32 * MAX_SEG), ("seg_len", C.c_int32 * MAX_SEG),
        ("seg_pack_off", C.c_int32 * MAX_SEG), ("seg_lut_off", C.c_int32 * MAX_SEG),
        ("lut_off", C.c_float * MAX_SEG), ("lut_inv", C.c_float * MAX_SEG),
        ("v_cents", C.c_float * 16), ("v_bounds", C.c_float * 16),
        ("v_lut", C.c_uint16 * 16), ("codebook", C.c_uint16 * 512), ("k_cents", C.c_float * 512),
        ("head_perm", C.c_uint8 * HD), ("group_of", C.c_uint8 * HD),
        ("code_lut", (C.c_uint8 * N_BINS) * MAX_SEG),
    ]


class DecodePlan(C.Structure):
    _fields_ = [("opaque", C.c_uint8 * 4096)]


_i32, _i64, _f32, _vp = C.c_int32, C.c_int64, C.c_float, C.c_void_p
_SIGNATURES = {
    "bgtq_abi_version": (C.c_int, []),
    "bgtq_desc_size": (C.c_int, []),
    "bgtq_error_string": (C.c_char_p, [C.c_int]),
    "bgtq_encode_tcgen05_status": (C.c_int, []),
    "bgtq_prefill_tcgen05_status": (C.c_int, []),
    "bgtq_encode": (C.c_int, [_vp, _vp, _vp,
                              _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64,
                              _i32, _i32, _i32, _i32,
                              _vp, _i64, _i64, _i64, _i32,
                              _vp, _i64, _i64, _i64, _i32,
                              _vp, _i64, _i64, _i64,
                              _vp, _i64, _i64, _i64,
                              _vp, _vp, _i32, _vp, _i32, _vp, _vp]),
    "bgtq_step_prepare_ring": (C.c_int, [_vp, _vp, _vp, _vp, _i64, _i64, _vp, _i32,
                                    _vp, _i64, _i64, _vp, _i64, _i64, _i32, _i32, _i32,
                                    _vp, _i64, _i64, _i64, _i32, _vp, _i64, _i64, _i64, _i32,
                                    _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64, _i32, _vp, _i32, _vp,
                                    _vp, _vp, _i64, _i64, _i32, _i32, _vp]),
    "bgtq_step_prepare_rope": (C.c_int, [_vp, _vp, _vp, _vp, _i64, _i64, _vp, _i32,
                                    _vp, _i64, _i64, _vp, _i64, _i64, _i32, _i32, _i32,
                                    _vp, _i64, _i64, _i64, _i32, _vp, _i64, _i64, _i64, _i32,
                                    _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64, _i32, _vp, _i32, _vp, _vp, _vp, _i64, _vp]),
    "bgtq_step_prepare": (C.c_int, [_vp, _vp, _vp, _vp, _i64, _i64, _vp, _i32,
                                    _vp, _i64, _i64, _vp, _i64, _i64, _i32, _i32, _i32,
                                    _vp, _i64, _i64, _i64, _i32, _vp, _i64, _i64, _i64, _i32,
                                    _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64, _i32, _vp, _i32, _vp, _vp]),
    "bgtq_rotate_q": (C.c_int, [_vp, _vp, _vp, _i64, _i64, _vp, _i32, _i32, _i32, _vp]),
    "bgtq_decode_plan": (C.c_int, [_vp, _i32, _i32, _vp]),
    "bgtq_decode_default_splits": (C.c_int, [_i32, _i32, _i32]),
    "bgtq_decode_image_bytes": (C.c_int64, [_vp]),
    "bgtq_decode_build_image": (C.c_int, [_vp, _vp, _vp, _i64]),
    "bgtq_decode_plan_set_image": (C.c_int, [_vp, _vp]),
    "bgtq_decode_plan_set_partition": (C.c_int, [_vp, _vp]),
    "bgtq_decode_plan_set_early_fetch": (C.c_int, [_vp, _i32]),
    "bgtq_decode_plan_set_row_strides": (C.c_int, [_vp, _i32, _i32, _i32, _i32]),
    "bgtq_decode_grid_size": (C.c_int, [_i32, _i32, _i32]),
    "bgtq_decode_partition": (C.c_int, [_i32, _i32, _i32, _i32, _i32, _vp, _i32]),
    "bgtq_decode_plan_specialize": (C.c_int, [_vp, _i32, C.c_char_p, _i64]),
    "bgtq_jit_set_nvrtc_path": (C.c_int, [C.c_char_p]),
    "bgtq_decode": (C.c_int, [_vp, _vp, _vp,
                              _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64,
                              _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64,
                              _i32, _i32, _i32, _i32, _i32, _i32, _f32,
                              _vp, _vp, _vp, _vp, _i32, _vp]),
    "bgtq_decode_combined_noalloc": (C.c_int, [_vp, _vp, _vp,
                                               _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64,
                                               _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64,
                                               _i32, _i32, _i32, _i32, _i32, _i32, _f32,
                                               _vp, _vp, _i64, _i64, _vp, _vp, _vp]),
    "bgtq_buffer_attn_pos": (C.c_int, [_vp, _i64, _i64, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _i32, _i32,
                                   _i32, _i32, _i32, _f32,
                                   _vp, _vp, _vp, _vp]),
    "bgtq_buffer_attn": (C.c_int, [_vp, _i64, _i64, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _i32, _i32,
                                   _i32, _i32, _i32, _f32,
                                   _vp, _vp, _vp]),
    "bgtq_prefill_attention": (C.c_int, [_vp, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64,
                                         _vp, _i64, _i64, _i64, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32,
                                         _i32, _i32, C.c_float, _i32, _vp, _vp]),
    "bgtq_combine_publish": (C.c_int, [_vp, _vp, _i32, _vp, _i32, _i32, _i32, _vp, _i64, _i64, _vp, _i32, _i32, _vp, _vp,
                                      _i32, _vp]),
    "bgtq_exchange_publish": (C.c_int, [_vp, _i64, _vp, _i64, _i64, _vp, _i32, _i32, _vp, _vp, _vp]),
    "bgtq_exchange_merge": (C.c_int, [_vp, _i32, _i64, _i64, _vp, _vp, _i32, _i32, _vp, _i64, _i64, _vp, _vp, _vp]),
    "bgtq_combine_ranks": (C.c_int, [_vp, _i32, _i64, _i32, _i32, _vp, _i64, _i64, _i32, _vp]),
    "bgtq_combine": (C.c_int, [_vp, _vp, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _i64, _i64, _vp, _vp, _i32, _vp]),
}

_lib = None
launches = 0          # kernels enqueued through this binding (read by the benchmark)


def exported_symbols():
    return sorted(_SIGNATURES)


def lib():
    """Load (building first if the sources are newer) and type the library."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB
    if _build.needs_build():
        path = _build.build()
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing and could not be built; the CUDA library is required")
    handle = C.CDLL(path)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(handle, name)
        fn.restype, fn.argtypes = res, args
    if handle.bgtq_desc_size() != C.sizeof(HeadDesc):
        raise RuntimeError(f"BgtqHeadDesc size mismatch: library {handle.bgtq_desc_size()} vs binding "
                           f"{C.sizeof(HeadDesc)}")
    _lib = handle
    return _lib


def check(code: int, what: str):
    if code != OK:
        raise RuntimeError(f"{what} failed: {lib().bgtq_error_string(code).decode()} ({code})")


def ptr(t):
    return 0 if t is None else t.data_ptr()


def stream_ptr(device=None):
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(t: torch.Tensor, name: str):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this package has no CPU path")


def count_launch(n=1):
    global launches
    launches += n
