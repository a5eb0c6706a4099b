"""ctypes binding of libxg_sm100.so (the C ABI declared in include/xg_sm100.h).

The library is loaded lazily and only from this package's directory. There is no fallback: if the
shared object is missing, fails to load, or lacks a symbol, ``XgLibraryError`` is raised and every
op that needs it fails loudly.
"""
from __future__ import annotations

import contextlib
import ctypes
import os
import threading
from ctypes import POINTER, c_char_p, c_float, c_int, c_int64, c_uint, c_uint8, c_void_p

LIB_NAME = "libxg_sm100.so"
LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), LIB_NAME)

XG_OK = 0
XG_F32, XG_BF16, XG_F16 = 0, 1, 2
ACT_CODES = {"none": 0, "gelu": 1, "relu": 2, "silu": 3, "sigmoid": 4}
ERR_NAMES = {-1: "INVALID_ARG", -2: "UNSUPPORTED", -3: "LAUNCH", -4: "DEVICE", -5: "TOO_LARGE"}


class XgLibraryError(RuntimeError):
    """The kernel library could not be loaded or a call into it failed."""


_I64P = POINTER(c_int64)
_VPP = POINTER(c_void_p)

# name -> (restype, argtypes); mirrors include/xg_sm100.h one to one.
SIGNATURES = {
    "xg_version": (c_int, []),
    "xg_device_arch_ok": (c_int, [c_int]),
    "xg_last_error": (c_char_p, []),
    "xg_tc_status": (c_int, [POINTER(c_uint), c_int]),
    "xg_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                           c_float, c_int, c_int, c_void_p]),
    "xg_layernorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                             c_int64, c_float, c_int, c_int, c_void_p]),
    "xg_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                        c_int64, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "xg_swiglu": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "xg_gemm_bias_act": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                 c_int64, c_int64, c_int64, c_int, c_int, c_int, c_void_p]),
    "xg_gemm_bias_act_ws": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                    c_int64, c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_int64, c_void_p]),
    "xg_gemm_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64, c_int]),
    "xg_gemm_bias_act_cluster": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                         c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p]),
    "xg_gemm_cluster_plan": (c_int, [c_int64, c_int64, c_int64, c_int, POINTER(c_int), POINTER(c_int)]),
    "xg_gemm_bias_act_static": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                        c_int64, c_int64, c_int64, c_int, c_int, c_int, c_void_p]),
    "xg_gemm_static_scratch_bytes": (c_int64, []),
    "xg_bgemm_bias_act": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                  c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                  c_int, c_int, c_int, c_void_p]),
    "xg_gemm_group_bias_act": (c_int, [_VPP, _VPP, _VPP, _VPP, _VPP, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                       c_int64, c_int64, c_int, c_int, c_int, c_void_p]),
    "xg_mlp_small_supported": (c_int, [_I64P, c_int, c_int]),
    "xg_mlp_small_bias_act": (c_int, [c_void_p, _VPP, _VPP, c_void_p, c_int64, _I64P, c_int, c_int64, _I64P, c_int64,
                                      POINTER(c_int), c_int, c_int, c_void_p]),
    "xg_mlp2_supported": (c_int, [c_int64, c_int64, c_int64, c_int64, c_int]),
    "xg_mlp3_supported": (c_int, [c_int64, c_int64, c_int64, c_int64, c_int64, c_int]),
    "xg_mlp3_bias_act": (c_int, [c_void_p] * 8 + [c_int64] * 10 + [c_int] * 5 + [c_void_p]),
    "xg_mlp2_bias_act": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                 c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p]),
    "xg_gemm_swiglu": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                               c_int64, c_int, c_void_p]),
    "xg_gemm_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                             c_int64, c_int64, c_int64, c_int, c_void_p]),
    "xg_sdpa_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                            c_int64, _I64P, _I64P, _I64P, _I64P, _I64P, c_float, c_int, c_int, c_void_p]),
    "xg_seg_copy": (c_int, [_VPP, _VPP, _I64P, _I64P, _I64P, c_int64, c_int64, c_void_p, c_int, c_void_p]),
    "xg_gemm_f32x3_padded_k": (c_int64, [c_int64]),
    "xg_split_bf16x3": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "xg_gemm_f32x3": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                              c_int, c_int, c_void_p]),
    "xg_sum3d": (c_int, [_VPP, _VPP, _I64P, c_int64, c_int, c_int, c_void_p]),
    "xg_rowsum_cat": (c_int, [_VPP, _VPP, _I64P, _I64P, _I64P, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int, c_void_p]),
    "xg_gather_rows": (c_int, [_VPP, _I64P, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int, c_void_p, c_int64,
                               c_int64, c_int64, c_int, c_void_p]),
}

_lock = threading.Lock()
_lib = None


def load(path: str | None = None) -> ctypes.CDLL:
    """Load the library (once) and bind every declared symbol. Raises XgLibraryError on any problem."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    with _lock:
        if _lib is not None and path is None:
            return _lib
        p = path or LIB_PATH
        if not os.path.exists(p):
            raise XgLibraryError(
                f"{p} not found: build it with `python -m xpu_graph_b200.build` (nvcc, sm_100a). "
                "The cuda_sm100 target has no fallback implementation."
            )
        try:
            lib = ctypes.CDLL(p)
        except OSError as e:  # pragma: no cover - depends on the environment
            raise XgLibraryError(f"cannot load {p}: {e}") from e
        for name, (res, args) in SIGNATURES.items():
            try:
                fn = getattr(lib, name)
            except AttributeError as e:
                raise XgLibraryError(f"{p} does not export {name}") from e
            fn.restype = res
            fn.argtypes = args
        if path is None:
            _lib = lib
        return lib


def last_error() -> str:
    msg = load().xg_last_error()
    return msg.decode() if msg else ""


def check(rc: int, what: str) -> None:
    if rc != XG_OK:
        raise XgLibraryError(f"{what} failed: {ERR_NAMES.get(rc, rc)}: {last_error()}")


def i64_array(values) -> "ctypes.Array":
    vals = [int(v) for v in values]
    return (c_int64 * len(vals))(*vals)


def ptr_array(values) -> "ctypes.Array":
    vals = [int(v) for v in values]
    return (c_void_p * len(vals))(*vals)


def tc_status(reset: bool = True) -> int:
    """Device status word of the tensor-core kernels (0 = healthy). Synchronises the device."""
    out = c_uint(0)
    check(load().xg_tc_status(ctypes.byref(out), 1 if reset else 0), "xg_tc_status")
    return int(out.value)


# entry points that enqueue no kernel (queries and status reads)
QUERY_ENTRY_POINTS = frozenset({"xg_version", "xg_device_arch_ok", "xg_last_error", "xg_tc_status", "xg_gemm_workspace_bytes",
                                "xg_gemm_static_scratch_bytes", "xg_gemm_f32x3_padded_k", "xg_gemm_cluster_plan",
                                "xg_mlp2_supported", "xg_mlp3_supported", "xg_mlp_small_supported"})


@contextlib.contextmanager
def call_hook(before=None, after=None):
    """While active, every call into the library made through ``load()`` is reported: ``before(name, args)`` just
    before the C function runs and ``after(name, args, rc)`` just after it returned (both optional; ``args`` are the
    marshalled arguments in the header's order). For observers that live outside the ops - launch counters, timers
    that bracket a kernel with events on the launching stream, call logs. Not thread-safe; do not nest."""
    lib = load()
    saved = {}
    for name in SIGNATURES:
        fn = getattr(lib, name)
        saved[name] = fn

        def wrapped(*args, _fn=fn, _name=name):
            if before is not None:
                before(_name, args)
            rc = _fn(*args)
            if after is not None:
                after(_name, args, rc)
            return rc

        setattr(lib, name, wrapped)
    try:
        yield lib
    finally:
        for name, fn in saved.items():
            setattr(lib, name, fn)
