"""ctypes binding of ``libsplinekv_b200.so`` (declared in ``include/splinekv_b200.h``)."""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libsplinekv_b200.so")

SKV_BF16, SKV_F32 = 0, 1
SKV_ACT = {"relu_sq": 0, "identity": 1, "gelu": 2}
SKV_IMPL = {"auto": 0, "simt": 1, "tcgen05": 2}
SKV_OP_FORWARD, SKV_OP_BACKWARD = 0, 1

EXPORTS = (
    "skv_abi_version", "skv_error_string", "skv_device_ok", "skv_resolve_impl", "skv_scratch_bytes",
    "skv_feature_forward", "skv_feature_backward", "skv_knot_index", "skv_kernel_launches",
    "skv_feature_forward_noalloc", "skv_debug_set", "skv_readout_scratch_bytes", "skv_feature_readout_forward",
)
SKV_DEBUG_WAIT_CYCLES, SKV_DEBUG_SKIP_FIRST_COPY, SKV_DEBUG_FUSED_BACKWARD = 0, 1, 2
SKV_NOALLOC_SCRATCH_BYTES = 16 << 20


class Problem(ctypes.Structure):
    """Mirror of ``struct skv_problem``."""
    _fields_ = [
        ("N", ctypes.c_int64), ("h", ctypes.c_int32), ("L", ctypes.c_int32), ("r", ctypes.c_int32),
        ("grid_lo", ctypes.c_float), ("scale", ctypes.c_float), ("lambda_scale", ctypes.c_float),
        ("activation", ctypes.c_int32), ("dtype", ctypes.c_int32), ("impl", ctypes.c_int32),
        ("delta_f32", ctypes.c_int32), ("dz_f32", ctypes.c_int32), ("spline_order", ctypes.c_int32),
    ]


class SplineKVError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"splinekv_b200 error {code}: {text}")
        self.code = code


_lib = None


def load() -> ctypes.CDLL:
    """Load the CUDA library; raise if it has not been built (there is no fallback path)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m sparsespline_ffn_b200.build` "
            "(needs nvcc with sm_100a support). This package has no CPU or eager fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    pp = ctypes.POINTER(Problem)
    lib.skv_abi_version.restype = i32
    lib.skv_error_string.argtypes = [i32]
    lib.skv_error_string.restype = ctypes.c_char_p
    lib.skv_device_ok.restype = i32
    lib.skv_resolve_impl.argtypes = [pp]
    lib.skv_resolve_impl.restype = i32
    lib.skv_scratch_bytes.argtypes = [pp, i32]
    lib.skv_scratch_bytes.restype = ctypes.c_size_t
    lib.skv_feature_forward.argtypes = [pp, vp, i64, vp, vp, i64, vp, i64, vp, ctypes.c_size_t, vp, vp]
    lib.skv_feature_forward.restype = i32
    lib.skv_feature_backward.argtypes = [pp, vp, i64, vp, vp, i64, vp, i64, vp, i64, vp, vp, vp,
                                         ctypes.c_size_t, vp, vp]
    lib.skv_feature_backward.restype = i32
    lib.skv_knot_index.argtypes = [pp, vp, i64, vp, vp]
    lib.skv_knot_index.restype = i32
    lib.skv_kernel_launches.restype = ctypes.c_uint64
    lib.skv_feature_forward_noalloc.argtypes = [pp, vp, i64, vp, vp, i64, vp, i64, vp, vp]
    lib.skv_feature_forward_noalloc.restype = i32
    lib.skv_debug_set.argtypes = [i32, i64]
    lib.skv_debug_set.restype = i32
    lib.skv_readout_scratch_bytes.argtypes = [pp, i64]
    lib.skv_readout_scratch_bytes.restype = ctypes.c_size_t
    lib.skv_feature_readout_forward.argtypes = [pp, vp, i64, vp, vp, i64, i64, vp, i64, vp, ctypes.c_size_t, vp, vp]
    lib.skv_feature_readout_forward.restype = i32
    if lib.skv_abi_version() != 4:
        raise RuntimeError("libsplinekv_b200.so has an unexpected ABI version; rebuild it")
    _lib = lib
    return lib


def check(code: int) -> None:
    if code != 0:
        raise SplineKVError(code, load().skv_error_string(code).decode())
