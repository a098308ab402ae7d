"""ctypes binding of ``libdpk_b200.so`` (the C ABI declared in ``include/dpk_b200.h``).

There is no fallback: if the library is missing or a call fails, an exception is
raised.  ``ValueError`` for rejected arguments, ``RuntimeError`` for CUDA failures
and for problems a kernel reported in its status word.
"""

from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_PKG), "lib", "libdpk_b200.so")

OK, ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_DEVICE = 0, 1, 2, 3, 4
F16, BF16 = 0, 1
ACT = {"identity": 0, "relu": 1, "silu": 2}

_vp, _i64, _i32, _sz, _f32 = C.c_void_p, C.c_int64, C.c_int, C.c_size_t, C.c_float

# name -> (restype, argtypes); every symbol include/dpk_b200.h declares
SIGNATURES = {
    "dpk_version": (_i32, []),
    "dpk_set_sm_margin": (_i32, [_i32]),
    "dpk_last_error": (C.c_char_p, []),
    "dpk_device_status": (_i32, [C.POINTER(_i32), _vp]),
    "dpk_topk_mask": (_i32, [_vp, _i64, _i32, _i32, _vp, _vp]),
    "dpk_route_workspace_bytes": (_sz, [_i32, _i64, _i32]),
    "dpk_route_compact": (_i32, [_vp, _i32, _i64, _i32, _vp, _vp, _vp, _vp, _sz, _vp]),
    "dpk_route_compact_static": (_i32, [_vp, _i32, _i64, _i32, _vp, _vp, _vp, _vp]),
    "dpk_route_counts": (_i32, [_vp, _i32, _i64, _i32, _vp, _vp]),
    "dpk_mask_pack": (_i32, [_vp, _i64, _i32, _vp, _vp, _vp]),
    "dpk_route_plan": (_i32, [_vp, _i64, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "dpk_gemm_mn": (_i32, [_vp, _i64, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32,
                           _i32, _i32, _vp]),
    "dpk_set_gemm_mn_gather": (_i32, [_i32]),
    "dpk_set_router_norm_cluster": (_i32, [_i32]),
    "dpk_set_gemm_k_wave_order": (_i32, [_i32]),
    "dpk_gemm_k": (_i32, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _i32,
                          _vp, _i64, _vp, _sz, _vp]),
    "dpk_gemm_k_workspace_bytes": (_sz, [_i64, _i32]),
    "dpk_gemv_routed": (_i32, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _i32,
                               _i32, _i32, _vp]),
    "dpk_ffn_workspace_bytes": (_sz, [_i64, _i32, _i32, _i32]),
    "dpk_ffn_swiglu": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _vp, _sz,
                              _vp]),
    "dpk_attn_prefill": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32,
                                _i32, _i32, _f32, _i32, _i32, _i32, _i64, _i64, _i64, _i64, _vp]),
    "dpk_set_attn_prefill_heads": (_i32, [_i32]),
    "dpk_attn_decode_workspace_bytes": (_sz, [_i32, _i32, _i32, _i32, _i32, _i32]),
    "dpk_attn_decode": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32,
                               _f32, _i32, _i64, _i64, _vp, _sz, _vp]),
    "dpk_ffn_small_workspace_bytes": (_sz, [_i64, _i32, _i32]),
    "dpk_ffn_swiglu_small": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _vp,
                                    _sz, _vp]),
    "dpk_router_norm": (_i32, [_vp, _i64, _vp, _f32, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _i64,
                               _i32, _i32, _i32, _i32, _i32, _vp]),
    "dpk_rope_append": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _i32, _i32, _i32, _i32, _i32,
                               _i64, _i64, _i32, _i64, _i64, _vp]),
    "dpk_peer_barrier": (_i32, [C.POINTER(_vp), _vp, _i32, _i32, C.c_uint32, _i32, _vp]),
    "dpk_peer_alloc": (_i32, [_sz, C.POINTER(_vp), _vp]),
    "dpk_peer_open": (_i32, [_vp, C.POINTER(_vp)]),
    "dpk_peer_close": (_i32, [_vp]),
    "dpk_peer_free": (_i32, [_vp]),
    "dpk_gemm_k_scatter_workspace_bytes": (_sz, [_i64, _i32, _i64]),
    "dpk_gemm_k_scatter": (_i32, [_vp, _i64, _vp, _i64, _vp, _vp, C.POINTER(_vp), _i32, _i32, _i64,
                                  _i64, _i64, _i32, _i32, _i32, _i32, _vp, _sz, _vp]),
    "dpk_reduce_gather": (_i32, [_vp, C.POINTER(_vp), _vp, _i32, _i32, _i64, _i64, _i32, _i64, _i32,
                                 _i32, _vp]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m dpk_b200.build` "
                "(there is no fallback implementation)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error() -> str:
    return load().dpk_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    if rc == OK:
        return
    msg = last_error()
    if rc in (ERR_INVALID, ERR_UNSUPPORTED):
        raise ValueError(f"dpk_b200: {msg}")
    raise RuntimeError(f"dpk_b200 (code {rc}): {msg}")


def device_status(stream_ptr: int) -> int:
    """Synchronise the stream and return the kernels' status word (0 = fine)."""
    out = _i32(0)
    check(load().dpk_device_status(C.byref(out), stream_ptr))
    return out.value
