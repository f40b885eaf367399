"""ctypes binding of libnsa_b200.so (the C ABI declared in include/nsa_b200.h).

There is no fallback: if the library is missing it is built with nvcc, and if that fails
the import raises.  Every wrapper raises RuntimeError with the library's own message on
a non-zero status.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libnsa_b200.so")

OK = 0
ABI_VERSION = 7      # nsa_abi_version() of the library these struct mirrors and prototypes describe
BF16, FP16, FP8_E4M3, FP8_E5M2, FP32 = 0, 1, 2, 3, 4
BRANCH_COMPRESSED, BRANCH_SELECTED, BRANCH_SLIDING = 1, 2, 4
GATE_SIGMOID, GATE_SOFTMAX = 0, 1
ENGINE_AUTO, ENGINE_GENERIC, ENGINE_TCGEN05 = 0, 1, 2
IO_OUT_BTHD, IO_GATES_BTHD = 1, 2

_DTYPE_CODE = {
    torch.bfloat16: BF16, torch.float16: FP16, torch.float32: FP32,
    torch.float8_e4m3fn: FP8_E4M3, torch.float8_e5m2: FP8_E5M2,
}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}") from None


class FwdArgs(C.Structure):
    """Mirror of `struct nsa_fwd_args`."""
    _fields_ = [
        ("Q", C.c_void_p), ("K", C.c_void_p), ("V", C.c_void_p), ("Kc", C.c_void_p), ("Vc", C.c_void_p),
        ("idx", C.c_void_p), ("gates", C.c_void_p), ("out", C.c_void_p), ("lse", C.c_void_p),
        ("B", C.c_int32), ("H", C.c_int32), ("Hkv", C.c_int32), ("Hi", C.c_int32),
        ("Tq", C.c_int32), ("Tk", C.c_int32), ("D", C.c_int32),
        ("offset", C.c_int32),
        ("Nc", C.c_int32), ("cmp_block", C.c_int32), ("cmp_stride", C.c_int32), ("cmp_offset", C.c_int32),
        ("nq", C.c_int32), ("top_k", C.c_int32), ("bm", C.c_int32), ("bn", C.c_int32), ("sel_key_limit", C.c_int32),
        ("window", C.c_int32), ("causal", C.c_int32),
        ("branches", C.c_int32), ("fused", C.c_int32), ("gate_act", C.c_int32),
        ("q_dtype", C.c_int32), ("kv_dtype", C.c_int32), ("gate_dtype", C.c_int32),
        ("scale", C.c_float), ("q_scale", C.c_float), ("k_scale", C.c_float), ("v_scale", C.c_float),
        ("engine", C.c_int32), ("io_layout", C.c_int32),
        ("nsplit", C.c_int32), ("split_scratch", C.c_void_p), ("split_scratch_bytes", C.c_int64),
        ("dyn_len", C.c_void_p), ("accumulate", C.c_int32),
    ]


class BwdArgs(C.Structure):
    """Mirror of `struct nsa_bwd_args`."""
    _fields_ = [
        ("Q", C.c_void_p), ("K", C.c_void_p), ("V", C.c_void_p), ("dO", C.c_void_p),
        ("lse", C.c_void_p), ("delta", C.c_void_p), ("idx", C.c_void_p),
        ("dQ", C.c_void_p), ("dK_f", C.c_void_p), ("dV_f", C.c_void_p),
        ("B", C.c_int32), ("H", C.c_int32), ("Hkv", C.c_int32), ("Hi", C.c_int32),
        ("Tq", C.c_int32), ("Tk", C.c_int32), ("D", C.c_int32),
        ("nq", C.c_int32), ("top_k", C.c_int32), ("bm", C.c_int32), ("bn", C.c_int32), ("sel_key_limit", C.c_int32),
        ("offset", C.c_int32), ("causal", C.c_int32), ("dtype", C.c_int32), ("dq_dtype", C.c_int32),
        ("scale", C.c_float),
        ("branch", C.c_int32), ("window", C.c_int32),
        ("Nc", C.c_int32), ("cmp_block", C.c_int32), ("cmp_stride", C.c_int32), ("cmp_offset", C.c_int32),
        ("engine", C.c_int32), ("scratch", C.c_void_p), ("scratch_bytes", C.c_int64),
    ]


_vp, _i, _f, _i64 = C.c_void_p, C.c_int, C.c_float, C.c_int64

PROTOTYPES = {
    "nsa_last_error": (C.c_char_p, []),
    "nsa_abi_version": (_i, []),
    "nsa_pool_mean": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "nsa_pool_learned": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "nsa_moba_block_indices": (_i, [_vp, _vp, _vp] + [_i] * 13 + [_f, _i, _vp]),
    "nsa_select_blocks": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _i, _vp]),
    "nsa_cmp_block_scores": (_i, [_vp, _vp, _vp, _vp] + [_i] * 13 + [_f, _i, _i, _i, _i, _vp]),
    "nsa_cmp_block_scores_tc": (_i, [_vp, _vp, _vp, _vp, _vp] + [_i] * 13 + [_f, _i, _i, _i, _i, _vp]),
    "nsa_topk_from_scores": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "nsa_attention_fwd": (_i, [C.POINTER(FwdArgs), _vp]),
    "nsa_device_status": (_i, [_vp]),
    "nsa_debug_set_device_status": (_i, [_i, _i]),
    "nsa_compressed_attention_static": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp]),
    "launch_selected_attn_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "nsa_bwd_delta": (_i, [_vp, _vp, _vp, _i64, _i, _i, _vp]),
    "nsa_selected_bwd": (_i, [C.POINTER(BwdArgs), _vp]),
    "nsa_attention_bwd": (_i, [C.POINTER(BwdArgs), _vp]),
    "nsa_attention_bwd_scratch_bytes": (_i64, [C.POINTER(BwdArgs)]),
    "nsa_pool_mean_bwd": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "launch_selected_attn_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "nsa_combine": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _vp]),
    "nsa_fp8_absmax": (_i, [_vp, _i64, _i, _vp, _vp]),
    "nsa_fp8_quantize": (_i, [_vp, _vp, _i64, _i, _i, _f, _vp]),
    "nsa_fp8_dequantize": (_i, [_vp, _vp, _i64, _i, _f, _vp]),
    "nsa_cast_from_f32": (_i, [_vp, _vp, _i64, _i, _vp]),
    "nsa_rope_to_heads": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "nsa_cache_append": (_i, [_vp] * 7 + [_i] * 12 + [_vp]),
    "nsa_cache_append_dev": (_i, [_vp] * 7 + [_i] * 4 + [_vp] + [_i] * 7 + [_vp]),
    "nsa_select_blocks_cached": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _f, _i, _i, _i, _i, _vp]),
    "nsa_memcpy_2d": (_i, [_vp, C.c_size_t, _vp, C.c_size_t, C.c_size_t, C.c_size_t, _i, _vp]),
}

_lib = None


def load() -> C.CDLL:
    """Load (building first if needed) the shared library; raises if that is impossible."""
    global _lib
    if _lib is not None:
        return _lib
    from . import build as _build
    try:
        _build.build()               # returns at once when the stamp of the source hashes matches the built library
    except RuntimeError:
        if not os.path.exists(LIB_PATH):
            raise                    # nothing to load; with a library present (no nvcc on this machine) the ABI check decides
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)      # AttributeError if the symbol is missing
        fn.restype, fn.argtypes = res, args
    if lib.nsa_abi_version() != ABI_VERSION:
        raise RuntimeError(f"{LIB_PATH} has ABI version {lib.nsa_abi_version()}, this package expects {ABI_VERSION}: "
                           "rebuild with `python -m nsa_from_scratch_b200.build --force`")
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != OK:
        msg = load().nsa_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed (status {rc}): {msg}")


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()
