"""ctypes binding of the C ABI declared in include/fa_b200.h.

The library is loaded from the package directory.  There is no fallback: if
`libfa_b200.so` is missing the import of any operator raises, with the build
command in the message.
"""
from __future__ import annotations

import ctypes
import os

from .build import LIB_PATH

_c = ctypes
_vp, _i, _i64, _sz = _c.c_void_p, _c.c_int, _c.c_int64, _c.c_size_t

# name -> (restype, argtypes); every symbol include/fa_b200.h declares
SIGNATURES = {
    "fa_version": (_i, []),
    "fa_last_error": (_c.c_char_p, []),
    "fa_decode_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "fa_decode_workspace_init": (_i, [_vp, _sz, _vp]),
    "fa_decode_status": (_i, [_vp, _vp, _c.POINTER(_i)]),
    "fa_decode_set_tuning": (_i, [_i, _i, _i]),
    "fa_paged_decode_gqa_f16": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i64, _i, _i64, _vp, _sz, _vp]),
    "fa_paged_decode_gqa_f16_out_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i64, _i, _i64, _vp, _sz, _vp]),
    "fa_paged_decode_gqa_f16_static_scratch": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i64, _i, _i64, _vp]),
    "fa_decode_gqa_f16": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "fa_decode_sliding_window_gqa_f16": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "fa_decode_int8_kv_cache_gqa": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "fa_decode_varlen_f16": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "fa_decode_int8_gqa": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _sz, _vp]),
    "fa_rope_append_paged_f16": (_i, [_vp] * 12 + [_i, _i, _i, _i, _i, _i, _i64, _i, _vp]),
    "fa_add_rmsnorm_bf16": (_i, [_vp, _vp, _vp, _vp, _i64, _i, _c.c_float, _vp]),
    "fa_qk_norm_split_f16": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _c.c_float, _vp]),
    "fa_qkv_rope_append_f16": (_i, [_vp] * 13 + [_i, _i, _i, _i, _i, _c.c_float, _i64, _i, _vp]),
    "fa_silu_mul_bf16": (_i, [_vp, _vp, _i64, _i, _vp]),
    "fa_half_to_bf16": (_i, [_vp, _vp, _i64, _vp]),
    "fa_peer_alloc": (_i, [_sz, _c.POINTER(_vp), _c.POINTER(_vp), _c.POINTER(_vp), _vp, _vp]),
    "fa_peer_open": (_i, [_vp, _c.POINTER(_vp)]),
    "fa_peer_close": (_i, [_vp]),
    "fa_peer_free": (_i, [_vp, _vp, _vp]),
    "fa_peer_allreduce_sum_bf16": (_i, [_c.POINTER(_vp), _c.POINTER(_vp), _vp, _i, _i, _i64, _i64, _vp]),
    "fa_peer_allreduce_add_rmsnorm_bf16": (_i, [_c.POINTER(_vp), _c.POINTER(_vp), _vp, _i, _i, _i64, _i64, _i64, _i64,
                                                _i, _vp, _c.c_float, _vp]),
    "fa_peer_allgather": (_i, [_c.POINTER(_vp), _c.POINTER(_vp), _vp, _i, _i, _vp, _i64, _i64, _vp]),
    "fa_peer_status": (_i, [_vp, _vp, _c.POINTER(_i)]),
    "fa_peer_reset": (_i, [_vp, _vp, _vp]),
    "fa_peer_set_max_polls": (_i, [_c.c_uint]),
    "fa_prefill_set_impl": (_i, [_i]),
    "fa_prefill_status": (_i, [_vp, _c.POINTER(_i), _i]),
    "fa_prefill_dense_f16": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "fa_prefill_varlen_f16": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i64, _i, _i, _i, _i, _i, _vp]),
    "fa_prefill_varlen_f16_out_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i64, _i, _i, _i, _i, _i, _vp]),
    "fa_paged_decode_gqa_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i64, _i, _i64, _vp, _sz, _vp]),
    "fa_decode_gqa_bf16": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "fa_prefill_dense_bf16": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "fa_prefill_varlen_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i64, _i, _i, _i, _i, _i, _vp]),
    "fa_rope_append_paged_bf16": (_i, [_vp] * 12 + [_i, _i, _i, _i, _i, _i, _i64, _i, _vp]),
    "fa_qkv_rope_append_bf16": (_i, [_vp] * 13 + [_i, _i, _i, _i, _i, _c.c_float, _i64, _i, _vp]),
}

_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA library has not been built. "
            "Run `python -m flash_attn_v100_b200.build` (needs nvcc); there is no CPU fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    return load().fa_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(last_error() or f"fa_b200 call failed with status {rc}")
