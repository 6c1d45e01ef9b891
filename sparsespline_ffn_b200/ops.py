"""Tensor-level entry points over the C ABI: allocate outputs and scratch with torch, pass raw
device pointers and the current stream to ``libsplinekv_b200.so``.

These are the functions the autograd operators and the sharded wrappers call.  They never fall
back to eager PyTorch: a CPU tensor, a missing library or a non-B200 device raises.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_DTYPES = {torch.bfloat16: _lib.SKV_BF16, torch.float32: _lib.SKV_F32}
_status_words: dict[int, torch.Tensor] = {}


def grid_scale(grid_lo: float, grid_hi: float, G: int) -> float:
    """``G / (hi - lo)`` in double, as the reference's wrappers compute it
    (src/sparsespline_ffn/cuda_ext/__init__.py:551); the library rounds it to float32."""
    return float(G) / (float(grid_hi) - float(grid_lo))


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 the kernels write to when a bounded wait runs out (0 = healthy)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status_words.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = t
    return t


def check_status(device: torch.device) -> None:
    """Synchronise and raise if any kernel on ``device`` reported a timed-out wait."""
    v = int(status_word(device).item())
    if v != 0:
        status_word(device).zero_()
        raise RuntimeError(f"splinekv_b200 kernel reported device status {v:#x} (a bounded wait ran out)")


def _problem(z: torch.Tensor, C: torch.Tensor, grid_lo, grid_hi, G, activation, lambda_scale, impl,
             spline_order: int = 2) -> _lib.Problem:
    if z.dim() != 2:
        raise ValueError(f"z must be 2D [N, h], got {tuple(z.shape)}")
    if C.dim() != 3:
        raise ValueError(f"C must be 3D [h, L, r], got {tuple(C.shape)}")
    N, h = z.shape
    hC, L, r = C.shape
    if hC != h:
        raise ValueError(f"C[0]={hC} != h={h}")
    if spline_order not in (1, 2):
        raise ValueError(f"spline_order must be 1 or 2; got {spline_order}")
    if L != G + spline_order:
        raise ValueError(f"L={L} should equal G+spline_order={G + spline_order}")
    if not float(grid_hi) > float(grid_lo):
        raise ValueError(f"grid_hi {grid_hi} <= grid_lo {grid_lo}")
    if activation not in _lib.SKV_ACT:
        raise ValueError(f"activation {activation!r} is not supported by the sm_100a kernels "
                         f"(supported: {sorted(_lib.SKV_ACT)})")
    if impl not in _lib.SKV_IMPL:
        raise ValueError(f"impl must be one of {sorted(_lib.SKV_IMPL)}, got {impl!r}")
    if not z.is_cuda or not C.is_cuda:
        raise RuntimeError("CUDA-only: splinekv_b200 has no CPU path (z and C must be CUDA tensors)")
    if z.device != C.device:
        raise RuntimeError(f"z is on {z.device} but C is on {C.device}")
    if z.dtype not in _DTYPES:
        raise RuntimeError(f"unsupported dtype {z.dtype}: the sm_100a kernels take bfloat16 or float32")
    return _lib.Problem(N=N, h=h, L=L, r=r, grid_lo=float(grid_lo), scale=grid_scale(grid_lo, grid_hi, G),
                        lambda_scale=float(lambda_scale), activation=_lib.SKV_ACT[activation],
                        dtype=_DTYPES[z.dtype], impl=_lib.SKV_IMPL[impl], spline_order=int(spline_order))


_warned_slow: set[tuple] = set()


def _warn_if_slow_family(lib, p: _lib.Problem, z: torch.Tensor, aligned_fn) -> None:
    """One warning per shape when a large bf16 problem is about to run on the CUDA-core kernels
    (r not a multiple of 16, h not a multiple of 8, a pointer or stride that is not 16-byte
    aligned, ...): they are a correctness fallback, tens of times slower than the tcgen05 kernels."""
    if z.dtype != torch.bfloat16 or p.impl != _lib.SKV_IMPL["auto"] or p.N * p.h < (1 << 24):
        return
    aligned = bool(aligned_fn())
    if aligned and lib.skv_resolve_impl(ctypes.byref(p)) == _lib.SKV_IMPL["tcgen05"]:
        return
    key = (p.h, p.L, p.r, aligned)
    if key in _warned_slow:
        return
    _warned_slow.add(key)
    import warnings
    why = ("a tensor whose base address or row stride is not 16-byte aligned" if not aligned else
           f"a shape outside the tcgen05 kernels' range (h={p.h}, L={p.L}, r={p.r}: need r % 16 == 0, r <= 128, "
           "h % 8 == 0, L <= 64)")
    warnings.warn(f"splinekv_b200: {p.N} x {p.h} bf16 problem runs on the CUDA-core fallback kernels because of "
                  f"{why}; expect it to be tens of times slower", RuntimeWarning, stacklevel=3)


def _aligned16(*tensors) -> bool:
    for t in tensors:
        if t is None:
            continue
        if t.data_ptr() % 16 or (t.dim() == 2 and (t.stride(0) * t.element_size()) % 16):
            return False
    return True


def _rows(t: torch.Tensor) -> torch.Tensor:
    """A view or copy of a 2-D tensor with unit inner stride (any row stride is passed through)."""
    if t.dim() == 2 and t.stride(1) == 1 and t.stride(0) >= t.shape[1]:
        return t
    return t.contiguous()


def _ptr(t: torch.Tensor | None):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _scratch(lib, p: _lib.Problem, op: int, device) -> tuple[torch.Tensor | None, int]:
    need = int(lib.skv_scratch_bytes(ctypes.byref(p), op))
    if need == 0:
        return None, 0
    return torch.empty(need, dtype=torch.uint8, device=device), need


def resolve_impl(z, C, grid_lo, grid_hi, G, impl="auto") -> str:
    """Name of the kernel family the library would use for this problem: 'simt' or 'tcgen05'."""
    lib = _lib.load()
    p = _problem(z, C, grid_lo, grid_hi, G, "relu_sq", 1.0, impl)
    code = lib.skv_resolve_impl(ctypes.byref(p))
    if code < 0:
        _lib.check(code)
    return {1: "simt", 2: "tcgen05"}[code]


def feature_forward(z, C, grid_lo, grid_hi, G, activation="relu_sq", lambda_scale=1.0, with_base=True,
                    impl="auto", out: torch.Tensor | None = None, delta_f32: bool = False, spline_order: int = 2):
    """``[phi(z); lambda*delta]`` as ``[N, h+r]`` (``with_base``) or ``lambda*delta`` as ``[N, r]``.

    With ``delta_f32`` the residual comes back in float32 whatever the dtype of ``z`` (the
    key-sharded mode sums partial residuals across GPUs before the one rounding to bf16); the two
    halves then cannot share a tensor, so the result is ``(phi(z) or None, delta_f32)``.
    ``spline_order=1`` selects the linear B-spline (``C`` is ``[h, G + 1, r]``; CUDA-core kernels)."""
    lib = _lib.load()
    C = C.to(z.dtype) if C.dtype != z.dtype else C
    p = _problem(z, C, grid_lo, grid_hi, G, activation, lambda_scale, impl, spline_order)
    z = _rows(z)
    C = C.contiguous()
    N, h, r = p.N, p.h, p.r
    p.delta_f32 = 1 if delta_f32 else 0
    with torch.cuda.device(z.device):
        if delta_f32:
            act = torch.empty((N, h), dtype=z.dtype, device=z.device) if with_base else None
            delta = torch.empty((N, r), dtype=torch.float32, device=z.device)
            act_ptr, act_stride = _ptr(act), h
            delta_ptr, delta_stride = _ptr(delta), r
            result = (act, delta)
        else:
            width = h + r if with_base else r
            f = out if out is not None else torch.empty((N, width), dtype=z.dtype, device=z.device)
            if tuple(f.shape) != (N, width) or f.dtype != z.dtype or f.stride(1) != 1:
                raise ValueError("out must be [N, width] in the dtype of z with unit inner stride")
            act_ptr = ctypes.c_void_p(f.data_ptr()) if with_base else None
            delta_ptr = ctypes.c_void_p(f.data_ptr() + (h * f.element_size() if with_base else 0))
            act_stride = delta_stride = f.stride(0)
            result = f
        _warn_if_slow_family(lib, p, z, lambda: _aligned16(z, C) and (delta_ptr.value or 0) % 16 == 0
                             and (delta_stride * (4 if delta_f32 else z.element_size())) % 16 == 0)
        scratch, nbytes = _scratch(lib, p, _lib.SKV_OP_FORWARD, z.device)
        code = lib.skv_feature_forward(
            ctypes.byref(p), _ptr(z), z.stride(0), _ptr(C), act_ptr, act_stride, delta_ptr, delta_stride,
            _ptr(scratch), nbytes, _ptr(status_word(z.device)),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(code)
    return result


def feature_readout_forward(z, C, W_out, grid_lo, grid_hi, G, activation="relu_sq", lambda_scale=1.0):
    """``y = [phi(z); lambda*delta] @ W_out.T`` as ``[N, d_out]`` without the feature in memory.

    bf16 only (``z``, ``C`` and ``W_out`` are cast as the reference's wrapper casts them,
    src/sparsespline_ffn/cuda_ext/__init__.py:626-632); ``W_out`` is ``[d_out, h + r]``, the layout of
    ``torch.nn.Linear.weight``.  Forward only."""
    lib = _lib.load()
    if not (z.is_cuda and C.is_cuda and W_out.is_cuda):
        raise RuntimeError("CUDA-only")
    z = z if z.dtype == torch.bfloat16 else z.to(torch.bfloat16)
    C = C if C.dtype == torch.bfloat16 else C.to(torch.bfloat16)
    W_out = W_out if W_out.dtype == torch.bfloat16 else W_out.to(torch.bfloat16)
    if activation not in ("relu_sq", "identity"):
        raise ValueError(f"unsupported activation: {activation}")
    p = _problem(z, C, grid_lo, grid_hi, G, activation, lambda_scale, "auto")
    if W_out.dim() != 2 or W_out.shape[1] != p.h + p.r:
        raise ValueError(f"W_out cols {tuple(W_out.shape)[-1]} != H+R={p.h + p.r}")
    z, C, W_out = z.contiguous(), C.contiguous(), W_out.contiguous()
    d_out = W_out.shape[0]
    with torch.cuda.device(z.device):
        y = torch.empty((p.N, d_out), dtype=torch.bfloat16, device=z.device)
        need = int(lib.skv_readout_scratch_bytes(ctypes.byref(p), d_out))
        if need == 0:
            raise ValueError(f"the fused read-out needs h, r and d_out to be multiples of 8; got h={p.h}, r={p.r}, "
                             f"d_out={d_out}")
        scratch = torch.empty(need, dtype=torch.uint8, device=z.device)
        code = lib.skv_feature_readout_forward(
            ctypes.byref(p), _ptr(z), z.stride(0), _ptr(C), _ptr(W_out), W_out.stride(0), d_out, _ptr(y), y.stride(0),
            _ptr(scratch), need, _ptr(status_word(z.device)),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(code)
    return y


def feature_backward(z, C, grad_out, grid_lo, grid_hi, G, activation="relu_sq", lambda_scale=1.0,
                     with_base=True, need_dz=True, need_dC=True, impl="auto", cast_dC=True, dz_f32=False,
                     spline_order: int = 2):
    """Gradients for ``grad_out`` of :func:`feature_forward`: one ``[N, h+r]`` (or ``[N, r]``) tensor,
    consumed in place through a base pointer and a row stride per half, or a ``(g_act, g_delta)``
    pair of separate tensors.

    Returns ``(dz or None, dC_f32 or None, dC_cast or None)``; ``dC_cast`` (dtype of ``C``) is only
    produced for bf16 problems when ``cast_dC`` is set.  ``dz_f32`` asks the tensor-core kernels of a
    bf16 problem for ``dz`` before its rounding to bf16 (a float32 tensor), which is how the tests
    measure a systematic error of ``dz``.
    """
    lib = _lib.load()
    C_in_dtype = C.dtype
    C = C.to(z.dtype) if C.dtype != z.dtype else C
    p = _problem(z, C, grid_lo, grid_hi, G, activation, lambda_scale, impl, spline_order)
    z = _rows(z)
    C = C.contiguous()
    N, h, r, L = p.N, p.h, p.r, p.L
    def _as_rows(t, cols, what):
        if tuple(t.shape) != (N, cols):
            raise ValueError(f"{what} must be [N, {cols}], got {tuple(t.shape)}")
        return _rows(t.to(z.dtype) if t.dtype != z.dtype else t)

    if isinstance(grad_out, (tuple, list)):
        # the two halves as separate tensors (each with its own row stride): nothing is concatenated
        if not with_base or len(grad_out) != 2:
            raise ValueError("a (g_act, g_delta) pair needs with_base=True and exactly two tensors")
        ga = _as_rows(grad_out[0], h, "g_act")
        gd = _as_rows(grad_out[1], r, "g_delta")
        gact_ptr, gact_stride = _ptr(ga), ga.stride(0)
        gdelta_ptr, gdelta_stride = _ptr(gd), gd.stride(0)
    else:
        go = _as_rows(grad_out, h + r if with_base else r, "grad_out")
        esz = go.element_size()
        gact_ptr = ctypes.c_void_p(go.data_ptr()) if with_base else None
        gdelta_ptr = ctypes.c_void_p(go.data_ptr() + (h * esz if with_base else 0))
        gact_stride = gdelta_stride = go.stride(0)
    with torch.cuda.device(z.device):
        p.dz_f32 = 1 if (dz_f32 and z.dtype != torch.float32) else 0
        dz = torch.empty((N, h), dtype=torch.float32 if dz_f32 else z.dtype, device=z.device) if need_dz else None
        dC = torch.empty((h, L, r), dtype=torch.float32, device=z.device) if need_dC else None
        dC_cast = None
        if need_dC and cast_dC and z.dtype != torch.float32:
            dC_cast = torch.empty((h, L, r), dtype=z.dtype, device=z.device)
        _warn_if_slow_family(lib, p, z, lambda: _aligned16(z, C) and (gdelta_ptr.value or 0) % 16 == 0
                             and (gact_ptr is None or (gact_ptr.value or 0) % 16 == 0)
                             and (gdelta_stride * z.element_size()) % 16 == 0
                             and (gact_stride * z.element_size()) % 16 == 0)
        scratch, nbytes = _scratch(lib, p, _lib.SKV_OP_BACKWARD, z.device)
        code = lib.skv_feature_backward(
            ctypes.byref(p), _ptr(z), z.stride(0), _ptr(C), gact_ptr, gact_stride, gdelta_ptr, gdelta_stride,
            _ptr(dz), h, _ptr(dC), _ptr(dC_cast), _ptr(scratch), nbytes, _ptr(status_word(z.device)),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(code)
    if dC_cast is not None and dC_cast.dtype != C_in_dtype:
        dC_cast = None
    return dz, dC, dC_cast


def knot_index(z, grid_lo, grid_hi, G) -> torch.Tensor:
    """int32 ``[N, h]`` knot-interval indices as the kernels compute them."""
    lib = _lib.load()
    if z.dim() != 2 or not z.is_cuda:
        raise ValueError("z must be a 2D CUDA tensor")
    if z.dtype not in _DTYPES:
        raise RuntimeError(f"unsupported dtype {z.dtype}")
    z = _rows(z)
    N, h = z.shape
    p = _lib.Problem(N=N, h=h, L=G + 2, r=1, grid_lo=float(grid_lo), scale=grid_scale(grid_lo, grid_hi, G),
                     lambda_scale=1.0, activation=0, dtype=_DTYPES[z.dtype], impl=1)
    with torch.cuda.device(z.device):
        bins = torch.empty((N, h), dtype=torch.int32, device=z.device)
        code = lib.skv_knot_index(ctypes.byref(p), _ptr(z), z.stride(0), _ptr(bins),
                                  ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(code)
    return bins
