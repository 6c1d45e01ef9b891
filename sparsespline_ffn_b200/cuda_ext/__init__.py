"""The two forward entry points of the reference's ``sparsespline_ffn.cuda_ext`` package, served by the
sm_100a library: same names, arguments, casts and errors
(src/sparsespline_ffn/cuda_ext/__init__.py:587-647), so that a benchmark or a model that imports them
from there can import them from here instead.
"""
from __future__ import annotations

import torch

from .. import ops


def spline_kv_fwd_cuda(z, C, grid_lo, grid_hi, G, activation: str = "relu_sq", lambda_scale: float = 1.0):
    """``f = [phi(z); lambda*delta]`` as ``[N, h + r]`` bf16."""
    if not (z.is_cuda and C.is_cuda):
        raise RuntimeError("CUDA-only")
    if activation not in {"relu_sq", "identity"}:
        raise ValueError(f"unsupported activation: {activation}")
    z = z if z.dtype == torch.bfloat16 else z.to(torch.bfloat16)
    C = C if C.dtype == torch.bfloat16 else C.to(torch.bfloat16)
    if z.dim() != 2 or C.dim() != 3 or C.shape[0] != z.shape[1] or C.shape[1] != G + 2:
        raise ValueError(f"shape mismatch: z={tuple(z.shape)} C={tuple(C.shape)} G={G}")
    return ops.feature_forward(z.contiguous(), C.contiguous(), grid_lo, grid_hi, G, activation, lambda_scale)


def spline_kv_fwd_fused_cuda(z, C, W_out, grid_lo, grid_hi, G, activation: str = "relu_sq",
                             lambda_scale: float = 1.0):
    """Fused forward + read-out: ``y = a @ W_out_a^T + lambda * delta @ W_out_d^T`` as ``[N, d_out]``,
    without the ``[N, h + r]`` feature tensor."""
    if not (z.is_cuda and C.is_cuda and W_out.is_cuda):
        raise RuntimeError("CUDA-only")
    if z.dim() != 2 or C.dim() != 3 or C.shape[0] != z.shape[1] or C.shape[1] != G + 2:
        raise ValueError(f"shape mismatch: z={tuple(z.shape)} C={tuple(C.shape)} G={G}")
    return ops.feature_readout_forward(z, C, W_out, grid_lo, grid_hi, G, activation, lambda_scale)


__all__ = ["spline_kv_fwd_cuda", "spline_kv_fwd_fused_cuda"]
