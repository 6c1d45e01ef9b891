"""ctypes binding and build recipe for the C restatement ``spline_kv_oracle.c``.

TEST INFRASTRUCTURE ONLY (see the header of ``spline_kv_oracle.c``): used by
``tests/``, by the smoke entry as the checker and by the benchmark's CPU
baseline.  The shipped package never imports this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "spline_kv_oracle.c")
_SO = os.path.join(_HERE, "libskv_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the C oracle next to its source (``gcc -O2 -fopenmp``)."""
    if (not force and os.path.exists(_SO)
            and os.path.getmtime(_SO) >= os.path.getmtime(_SRC)):
        return _SO
    cmd = ["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-shared", "-fPIC", _SRC, "-o", _SO]
    subprocess.run(cmd, check=True)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = ctypes.CDLL(_SO)
        fp = ctypes.POINTER(ctypes.c_float)
        dp = ctypes.POINTER(ctypes.c_double)
        ip = ctypes.POINTER(ctypes.c_int32)
        i64, i32, f32 = ctypes.c_int64, ctypes.c_int, ctypes.c_float
        L.skvo_num_threads.restype = ctypes.c_int
        L.skvo_set_threads.argtypes = [ctypes.c_int]
        L.skvo_set_threads.restype = None
        L.skvo_knot_index.argtypes = [fp, i64, i64, i32, f32, f32, i32, ip]
        L.skvo_knot_index.restype = None
        L.skvo_forward.argtypes = [fp, i64, fp, i64, i32, i32, i32, f32, f32, f32, i32, fp, fp]
        L.skvo_forward.restype = None
        L.skvo_backward.argtypes = [fp, i64, fp, fp, i64, fp, i64, i64, i32, i32, i32,
                                    f32, f32, f32, i32, fp, dp]
        L.skvo_backward.restype = None
        L.skvo_forward_o.argtypes = [fp, i64, fp, i64, i32, i32, i32, f32, f32, f32, i32, i32, fp, fp]
        L.skvo_forward_o.restype = None
        L.skvo_backward_o.argtypes = [fp, i64, fp, fp, i64, fp, i64, i64, i32, i32, i32,
                                      f32, f32, f32, i32, i32, fp, dp]
        L.skvo_backward_o.restype = None
        _lib = L
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a, t):
    return a.ctypes.data_as(ctypes.POINTER(t))


def _scale(grid_lo, grid_hi, G) -> float:
    return float(np.float32(float(G) / (float(grid_hi) - float(grid_lo))))


_ACT = {"relu_sq": 0, "identity": 1, "gelu": 2}


def num_threads() -> int:
    return int(lib().skvo_num_threads())


def set_threads(n: int) -> int:
    """Use ``n`` OpenMP threads from now on (launchers such as torch.distributed.run export
    OMP_NUM_THREADS=1, which would otherwise make this a one-core baseline); returns the count."""
    lib().skvo_set_threads(int(n))
    return num_threads()


def knot_index(z32, grid_lo, grid_hi, G) -> np.ndarray:
    z = _f32(z32)
    N, h = z.shape
    out = np.empty((N, h), dtype=np.int32)
    lib().skvo_knot_index(_p(z, ctypes.c_float), h, N, h, float(np.float32(grid_lo)),
                          _scale(grid_lo, grid_hi, G), G, _p(out, ctypes.c_int32))
    return out


def feature_forward(z32, C32, grid_lo, grid_hi, G, activation_name="relu_sq", lambda_scale=1.0,
                    want_activation=True, spline_order=2):
    """Returns ``(a [N,h] or None, lambda*delta [N,r])`` as float32 (``spline_order`` 2: quadratic,
    L = G + 2; 1: linear, L = G + 1)."""
    z = _f32(z32)
    C = _f32(C32)
    N, h = z.shape
    hC, L, r = C.shape
    if hC != h or L != G + spline_order or spline_order not in (1, 2):
        raise ValueError("shape mismatch")
    a = np.empty((N, h), dtype=np.float32) if want_activation else None
    d = np.empty((N, r), dtype=np.float32)
    lib().skvo_forward_o(_p(z, ctypes.c_float), h, _p(C, ctypes.c_float), N, h, L, r,
                         float(np.float32(grid_lo)), _scale(grid_lo, grid_hi, G),
                         float(lambda_scale), _ACT[activation_name], int(spline_order),
                         _p(a, ctypes.c_float) if a is not None else None, _p(d, ctypes.c_float))
    return a, d


def feature_backward(z32, C32, g_delta32, g_a32, grid_lo, grid_hi, G, activation_name="relu_sq",
                     lambda_scale=1.0, spline_order=2):
    """Returns ``(dz [N,h] float32, dC [h,L,r] float64)``; ``g_a32`` may be None."""
    z = _f32(z32)
    C = _f32(C32)
    gd = _f32(g_delta32)
    ga = _f32(g_a32) if g_a32 is not None else None
    N, h = z.shape
    _, L, r = C.shape
    dz = np.empty((N, h), dtype=np.float32)
    dC = np.empty((h, L, r), dtype=np.float64)
    lib().skvo_backward_o(_p(z, ctypes.c_float), h, _p(C, ctypes.c_float),
                          _p(gd, ctypes.c_float), r,
                          _p(ga, ctypes.c_float) if ga is not None else None, h,
                          N, h, L, r, float(np.float32(grid_lo)), _scale(grid_lo, grid_hi, G),
                          float(lambda_scale), _ACT[activation_name], int(spline_order),
                          _p(dz, ctypes.c_float), _p(dC, ctypes.c_double))
    return dz, dC


if __name__ == "__main__":
    print(build(force=True))
