"""ctypes binding of libtritonllm_b200.so (the C ABI declared in include/tritonllm_b200.h).

The library is the product: there is no Python or CPU fallback.  Loading fails
loudly when the shared object has not been built.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libtritonllm_b200.so")

_vp, _i64, _i32, _f32, _sz = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_size_t

# name -> (restype, argtypes); mirrors include/tritonllm_b200.h one to one
PROTOTYPES = {
    "b2_version": (_i32, []),
    "b2_status_string": (C.c_char_p, [_i32]),
    "b2_device_status": (_i32, [_i32, C.POINTER(_i32)]),
    "b2_set_tunable": (_i32, [C.c_char_p, _i32]),
    "b2_set_trace_buffer": (_i32, [_vp, _sz]),
    "b2_selftest_wait_timeout": (_i32, [_vp]),
    "b2_rmsnorm": (_i32, [_vp, _vp, _vp, _i64, _i32, _f32, _vp]),
    "b2_add_rmsnorm": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _f32, _vp]),
    "b2_rope_inplace": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _i64, _vp]),
    "b2_qkv_rope_kv_decode": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64,
                                     _i32, _i32, _i32, _i32, _i64, _vp]),
    "b2_qkv_rope_kv_decode_ragged": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp,
                                            _i64, _i32, _i64, _i32, _i32, _i32, _i32, _i64, _vp]),
    "b2_oproj_residual_decode": (_i32, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp]),
    "b2_linear_bias": (_i32, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp]),
    "b2_qkv_rope_prefill": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32,
                                   _i64, _i64, _i32, _i32, _i32, _i32, _i64, _i32, _vp]),
    "b2_oproj_residual": (_i32, [_vp, _i64, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i32, _i32, _vp]),
    "b2_router_logits": (_i32, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp]),
    "b2_attn_prefill": (_i32, [_vp, _vp, _vp, _vp, _i32, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _i64, _i64, _i64,
                               _f32, _i32, _vp, _i32, _vp]),
    "b2_attn_decode_workspace_bytes": (_sz, [_i64, _i32, _i32]),
    "b2_attn_decode": (_i32, [_vp, _vp, _vp, _vp, _i32, _vp, _i64, _i32, _i32, _i32, _i64, _i64, _i64, _i64, _f32,
                              _i32, _vp, _i32, _vp, _sz, _vp]),
    "b2_attn_decode_ragged": (_i32, [_vp, _vp, _vp, _vp, _i32, _vp, _i64, _i32, _i32, _i32, _i64, _i64, _i64, _i64, _f32,
                                     _i32, _vp, _i32, _vp, _i64, _i32, _i64, _vp, _sz, _vp]),
    "b2_attn_decode_static_max_units": (_sz, []),
    "b2_attn_decode_static": (_i32, [_vp, _vp, _vp, _vp, _i32, _vp, _i64, _i32, _i32, _i32, _i64, _i64, _i64, _i64,
                                     _f32, _i32, _vp, _i32, _vp]),
    "b2_mxfp4_upcast": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "b2_unembed_workspace_bytes": (_sz, [_i64, _i32]),
    "b2_unembed_decode": (_i32, [_vp, _i64, _vp, _vp, _i64, _vp, _vp, _sz, _i64, _i32, _i32, _vp]),
    "b2_moe_combine_add_rmsnorm": (_i32, [_vp, _sz, _i64, _i32, _i32, _vp, _i64, _vp, _f32, _vp, _i64, _vp, _i64, _vp]),
    "b2_norm_router_topk": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i32, _i32, _i32, _f32,
                                   _vp]),
    "b2_kv_slide": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp]),
    "b2_kv_zero_tail": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "b2_embed_gather": (_i32, [_vp, _i64, _vp, _i32, _vp, _i64, _i64, _i32, _i64, _vp]),
    "b2_moe_decode_workspace_bytes": (_sz, [_i64, _i32, _i32]),
    "b2_moe_fp4_workspace_bytes": (_sz, [_i64, _i32, _i32]),
    "b2_moe_experts_decode_fp4": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _sz, _i64, _i32,
                                         _i32, _i32, _f32, _f32, _vp]),
    "b2_moe_experts_decode": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _sz, _i64, _i32,
                                     _i32, _i32, _f32, _f32, _vp]),
    "b2_moe_prefill_workspace_bytes": (_sz, [_i64, _i32, _i32, _i32]),
    "b2_moe_upcast_packed": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "b2_moe_experts_prefill": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _sz, _i64, _i32, _i32, _i32,
                                      _f32, _f32, _vp]),
    "b2_swiglu": (_i32, [_vp, _i64, _vp, _i64, _i64, _i64, _f32, _f32, _vp]),
    "b2_topk_softmax": (_i32, [_vp, _i64, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _i64, _i64, _vp, _i32, _vp]),
}

_lib = None
_lock = threading.Lock()


class B2Error(RuntimeError):
    """A C-ABI entry point returned a non-zero status."""

    def __init__(self, fn: str, status: int, text: str):
        super().__init__(f"{fn} failed with status {status}: {text}")
        self.fn, self.status = fn, status


def load() -> C.CDLL:
    """Loads the shared library (once) and installs the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m tritonllm_b200.build` "
                "(needs nvcc); tritonllm_b200 has no fallback path")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)  # AttributeError here = header and library disagree
            fn.restype, fn.argtypes = res, args
        # TRITONLLM_B200_TUNE="name=value,name=value": tuning knobs applied once at load (unknown names are an error)
        for kv in filter(None, os.environ.get("TRITONLLM_B200_TUNE", "").split(",")):
            name, _, value = kv.partition("=")
            st = lib.b2_set_tunable(name.strip().encode(), int(value))
            if st != 0:
                raise RuntimeError(f"TRITONLLM_B200_TUNE: cannot set {kv!r} (status {st})")
        _lib = lib
    return _lib


def check(fn: str, status: int) -> None:
    if status != 0:
        text = load().b2_status_string(status)
        raise B2Error(fn, status, text.decode() if text else "?")


def call(fn: str, *args) -> None:
    """Calls a status-returning entry point and raises B2Error on failure."""
    check(fn, getattr(load(), fn)(*args))


def device_status(reset: bool = True) -> int:
    """The per-device status word (0 = no kernel has recorded a failure); synchronises the device.  The word is
    cleared only when it was non-zero, so the common case costs one 4-byte read."""
    out = _i32(0)
    check("b2_device_status", load().b2_device_status(0, C.byref(out)))
    if out.value and reset:
        check("b2_device_status", load().b2_device_status(1, C.byref(_i32(0))))
    return out.value
