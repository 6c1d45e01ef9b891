"""Autograd operators of the RL-Spline-KV feature path on B200.

Same classes, argument order and return structure as the reference's operator module
(``src/sparsespline_ffn/kernels/flash_spline_feature_autograd.py:30-292`` for
``FlashSplineFeature`` / ``flash_spline_feature`` and ``:295-444`` for ``FlashSplineDelta`` /
``flash_spline_delta``), so ``RLSplineKVReference.forward``
(``src/sparsespline_ffn/rl_spline_kv_reference.py:306-311, 328-333, 356-363``) can call them
unchanged.  What differs, on purpose:

* The reference's ``fwd_kernel`` x ``bwd_kernel`` dispatch over Triton and Hopper kernels is one
  sm_100a library.  The two strings are still accepted; every name of the reference's vocabulary
  means "the library's choice", and ``"simt"`` / ``"tcgen05"`` force a kernel family.  The
  ``SPARSE_SPLINE_FWD_KERNEL`` environment override is honoured the same way.
* There is no CPU and no eager path: ``use_kernel=False``, CPU tensors or a missing library raise
  ``RuntimeError`` instead of running PyTorch code.
* ``grad_output`` is consumed in place (no ``.contiguous()`` copies of its two halves) and the
  lambda chain-rule factor is applied inside the kernels in float32.
"""
from __future__ import annotations

import os

import torch

from .. import ops

# kernel names the reference accepts (flash_spline_feature_autograd.py:47-51, 83-131, 176-225)
_REFERENCE_FWD = {"auto", "triton", "wgmma_cuda", "v10_cuda", "v11_cuda"}
_REFERENCE_BWD = {"triton", "hopper_cuda", "wgmma_cuda", "wgmma_v5_cuda"}
_OURS = {"simt", "tcgen05"}


def _impl_of(name: str, vocabulary: set[str], what: str) -> str:
    if name in _OURS:
        return name
    if name in vocabulary:
        return "auto"
    raise ValueError(f"unknown {what} {name!r}; expected one of {sorted(vocabulary | _OURS)}")


def _require_kernel(use_kernel: bool, z: torch.Tensor) -> None:
    if not use_kernel:
        raise RuntimeError(
            "use_kernel=False asks for the PyTorch reference path, which this package does not ship "
            "(it has no eager fallback); call with use_kernel=True on CUDA tensors")
    if not z.is_cuda:
        raise RuntimeError("CUDA-only: the sm_100a kernels have no CPU path (z is a CPU tensor)")


def _capture_safe_dC_return(C: torch.Tensor, dC: torch.Tensor | None):
    """During CUDA-graph capture add into the preallocated ``C.grad`` and return None, as the
    reference does (flash_spline_feature_autograd.py:154-172): graph replay does not re-run the
    Python backward, so the accumulation must be part of the captured work."""
    if dC is None or not C.requires_grad:
        return None
    if C.grad is not None and torch.cuda.is_current_stream_capturing():
        C.grad.add_(dC.to(C.grad.dtype))
        return None
    return dC


class FlashSplineFeature(torch.autograd.Function):
    """``f = [phi(z); lambda * delta(z, C)]`` as ``[N, h + r]`` in the dtype of ``z``."""

    @staticmethod
    def forward(ctx, z, C, grid_lo, grid_hi, G, activation, lambda_scale, use_kernel,
                bwd_kernel="triton", fwd_kernel="auto"):
        chosen_fwd = os.environ.get("SPARSE_SPLINE_FWD_KERNEL", "") or fwd_kernel
        fwd_impl = _impl_of(chosen_fwd, _REFERENCE_FWD, "fwd_kernel")
        bwd_impl = _impl_of(bwd_kernel, _REFERENCE_BWD, "bwd_kernel")
        _require_kernel(use_kernel, z)
        f = ops.feature_forward(z.detach(), C.detach(), grid_lo, grid_hi, G, activation, lambda_scale,
                                with_base=True, impl=fwd_impl)
        ctx.save_for_backward(z, C)
        ctx.grid_lo = float(grid_lo)
        ctx.grid_hi = float(grid_hi)
        ctx.G = int(G)
        ctx.activation = activation
        ctx.lambda_scale = float(lambda_scale)
        ctx.bwd_impl = bwd_impl
        return f

    @staticmethod
    def backward(ctx, grad_output):
        z, C = ctx.saved_tensors
        need_dz, need_dC = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dz, dC32, dC_cast = ops.feature_backward(
            z.detach(), C.detach(), grad_output, ctx.grid_lo, ctx.grid_hi, ctx.G, ctx.activation,
            ctx.lambda_scale, with_base=True, need_dz=need_dz, need_dC=need_dC, impl=ctx.bwd_impl)
        dC = None
        if need_dC:
            dC = dC_cast if dC_cast is not None else dC32.to(C.dtype)
        return (dz, _capture_safe_dC_return(C, dC), None, None, None, None, None, None, None, None)


class SplineFeatureOfOrder(torch.autograd.Function):
    """``[phi(z); lambda * delta(z, C)]`` for a spline order given explicitly.  The reference's
    operators have no such argument (they are the quadratic spline; its linear spline,
    ``spline_order=1`` of ``flash_spline_feature_reference``, src/sparsespline_ffn/rl_spline_kv_reference.py:178-187,
    runs in PyTorch only), so this is a separate Function and :class:`FlashSplineFeature` keeps the
    reference's argument list."""

    @staticmethod
    def forward(ctx, z, C, grid_lo, grid_hi, G, activation, lambda_scale, spline_order):
        _require_kernel(True, z)
        f = ops.feature_forward(z.detach(), C.detach(), grid_lo, grid_hi, G, activation, lambda_scale,
                                with_base=True, spline_order=spline_order)
        ctx.save_for_backward(z, C)
        ctx.cfg = (float(grid_lo), float(grid_hi), int(G), activation, float(lambda_scale), int(spline_order))
        return f

    @staticmethod
    def backward(ctx, grad_output):
        z, C = ctx.saved_tensors
        lo, hi, G, act, lam, order = ctx.cfg
        need_dz, need_dC = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dz, dC32, dC_cast = ops.feature_backward(z.detach(), C.detach(), grad_output, lo, hi, G, act, lam,
                                                 with_base=True, need_dz=need_dz, need_dC=need_dC,
                                                 spline_order=order)
        dC = None
        if need_dC:
            dC = dC_cast if dC_cast is not None else dC32.to(C.dtype)
        return (dz, _capture_safe_dC_return(C, dC), None, None, None, None, None, None)


def flash_spline_feature(z, C, grid_lo=-3.0, grid_hi=3.0, G=20, activation="relu_sq", lambda_scale=1.0,
                         use_kernel=True, bwd_kernel="triton", fwd_kernel="auto", spline_order=2):
    """Functional form of :class:`FlashSplineFeature` (same defaults as the reference's wrapper,
    flash_spline_feature_autograd.py:269-292).  ``spline_order=1`` (not an argument of the reference's
    wrapper) selects the linear B-spline through :class:`SplineFeatureOfOrder`."""
    if spline_order != 2:
        _require_kernel(use_kernel, z)
        return SplineFeatureOfOrder.apply(z, C, grid_lo, grid_hi, G, activation, lambda_scale, spline_order)
    return FlashSplineFeature.apply(z, C, grid_lo, grid_hi, G, activation, lambda_scale, use_kernel,
                                    bwd_kernel, fwd_kernel)


class FlashSplineDelta(torch.autograd.Function):
    """Spline residual only: ``lambda * delta(z, C)`` as ``[N, r]``; no base path in either
    direction (reference: flash_spline_feature_autograd.py:295-429)."""

    @staticmethod
    def forward(ctx, z, C, grid_lo, grid_hi, G, lambda_scale, bwd_kernel):
        bwd_impl = _impl_of(bwd_kernel, _REFERENCE_BWD, "bwd_kernel")
        _require_kernel(True, z)
        delta = ops.feature_forward(z.detach(), C.detach(), grid_lo, grid_hi, G, "identity", lambda_scale,
                                    with_base=False, impl=bwd_impl if bwd_impl in _OURS else "auto")
        ctx.save_for_backward(z, C)
        ctx.grid_lo = float(grid_lo)
        ctx.grid_hi = float(grid_hi)
        ctx.G = int(G)
        ctx.lambda_scale = float(lambda_scale)
        ctx.bwd_impl = bwd_impl
        return delta

    @staticmethod
    def backward(ctx, grad_output):
        z, C = ctx.saved_tensors
        need_dz, need_dC = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dz, dC32, dC_cast = ops.feature_backward(
            z.detach(), C.detach(), grad_output, ctx.grid_lo, ctx.grid_hi, ctx.G, "identity",
            ctx.lambda_scale, with_base=False, need_dz=need_dz, need_dC=need_dC, impl=ctx.bwd_impl)
        dC = None
        if need_dC:
            dC = dC_cast if dC_cast is not None else dC32.to(C.dtype)
        return (dz, _capture_safe_dC_return(C, dC), None, None, None, None, None)


def flash_spline_delta(z, C, grid_lo=-3.0, grid_hi=3.0, G=20, lambda_scale=1.0, bwd_kernel="wgmma_cuda"):
    """Functional form of :class:`FlashSplineDelta` (flash_spline_feature_autograd.py:432-444)."""
    return FlashSplineDelta.apply(z, C, grid_lo, grid_hi, G, lambda_scale, bwd_kernel)


__all__ = ["FlashSplineFeature", "flash_spline_feature", "FlashSplineDelta", "flash_spline_delta",
           "SplineFeatureOfOrder"]
