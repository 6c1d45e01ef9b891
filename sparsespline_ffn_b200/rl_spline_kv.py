"""The RL-Spline-KV layer on top of this package's operators: ``y = W_out [phi(K x); lambda*delta(K x, C)]``.

Host-side mirror of the caller of the operator in the reference project
(``RLSplineKVConfig`` and ``RLSplineKVReference`` in ``src/sparsespline_ffn/rl_spline_kv_reference.py:30-75,
206-498``): the same configuration fields and validation, the same parameter and buffer names
(``K``, ``C``, ``W_out``, ``W_d_proj``, ``grid_lo_buf``, ``grid_hi_buf``), so that a state dict of the
reference module loads, and the same three forward graphs:

* additive (default):  ``f = FlashSplineFeature(z, C)``, ``y = W_out f``           (reference ``:351-364``)
* ``no_base``:          ``delta = FlashSplineDelta(z, C)``, ``y = W_out delta``     (``:299-315``)
* multiplicative gate:  ``y = W_out ((1 + W_d_proj delta) * phi(z))``               (``:316-350``)

What differs, on purpose: the operator always runs on the sm_100a kernels (there is no eager path, so
``use_kernel`` is accepted and must not be asked to be False on this package's behalf: a CPU input
raises), ``spline_order = 1`` (the linear spline, additive mode only, as in the reference, ``:303, 323``)
runs on the library's CUDA-core kernels instead of PyTorch code, and the per-forward diagnostics of the reference (``:376-481``) are not computed, which
also removes the host synchronisations they cause.  The two GEMMs around the operator are
``torch.nn.Linear``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .kernels.flash_spline_feature_autograd import FlashSplineDelta, FlashSplineFeature, SplineFeatureOfOrder


@dataclass
class RLSplineKVConfig:
    """Hyper-parameters of one layer; field names, defaults and checks follow the reference's
    dataclass (``rl_spline_kv_reference.py:30-75``)."""

    d: int
    h_ratio: float = 1.0
    r: int = 64
    G: int = 20
    spline_order: int = 2
    grid_lo: float = -3.0
    grid_hi: float = 3.0
    lambda_scale: float = 1.0
    activation: str = "relu_sq"
    bias: bool = False
    init_C_zero: bool = True
    use_kernel: bool = True
    bwd_kernel: str = "triton"
    fwd_kernel: str = "auto"
    no_base: bool = False
    gating_mode: str = "additive"
    c_init_std: float = 0.0

    def __post_init__(self) -> None:
        if self.G < 2:
            raise ValueError(f"G={self.G} too small")
        if self.grid_hi <= self.grid_lo:
            raise ValueError(f"grid_hi {self.grid_hi} <= grid_lo {self.grid_lo}")
        if not (0 < self.h_ratio <= 4):
            raise ValueError(f"h_ratio {self.h_ratio} outside (0, 4]")
        if self.r < 1:
            raise ValueError(f"r={self.r} must be >= 1")
        if self.spline_order not in (1, 2):
            raise ValueError(f"spline_order must be 1 or 2; got {self.spline_order}")
        if self.activation not in ("relu_sq", "gelu", "identity"):
            raise ValueError(f"unknown activation: {self.activation}")
        if self.gating_mode not in ("additive", "multiplicative"):
            raise ValueError(f"gating_mode must be 'additive' or 'multiplicative'; got {self.gating_mode}")
        if self.c_init_std < 0:
            raise ValueError(f"c_init_std must be >= 0; got {self.c_init_std}")
        if self.gating_mode == "multiplicative" and self.no_base:
            raise ValueError("multiplicative gating requires base path (no_base=True is incompatible)")


def _phi(z: torch.Tensor, name: str) -> torch.Tensor:
    if name == "relu_sq":
        return torch.where(z > 0, z * z, torch.zeros_like(z))
    if name == "gelu":
        return F.gelu(z)
    return z


class RLSplineKV(nn.Module):
    """One RL-Spline-KV feed-forward layer whose feature step runs on the sm_100a kernels."""

    def __init__(self, cfg: RLSplineKVConfig, operator_dtype: torch.dtype | None = None,
                 fused_readout: bool = False) -> None:
        """``operator_dtype``: run the feature operator in this dtype whatever the dtype of the
        module (z and C are cast on entry, the result is cast back), e.g. ``torch.bfloat16`` for the
        tensor-core kernels under float32 master weights and GEMMs; None keeps the dtype of ``K x``.
        ``fused_readout``: when no gradient is being recorded, the additive quadratic-spline graph with a
        ``relu_sq`` or ``identity`` base computes ``W_out f`` through the fused read-out (bf16, the feature
        tensor is never allocated; what the reference offers as ``spline_kv_fwd_fused_cuda``,
        ``src/sparsespline_ffn/cuda_ext/__init__.py:617-647``)."""
        super().__init__()
        self.operator_dtype = operator_dtype
        self.fused_readout = fused_readout
        if cfg.spline_order != 2 and (cfg.no_base or cfg.gating_mode == "multiplicative"):
            raise NotImplementedError("no_base and multiplicative gating require spline_order=2")
        self.cfg = cfg
        d = cfg.d
        h = max(1, int(d * cfg.h_ratio))
        self.h = h
        L = cfg.G + cfg.spline_order
        self.K = nn.Linear(d, h, bias=cfg.bias)
        self.C = nn.Parameter(torch.empty(h, L, cfg.r))
        if cfg.gating_mode == "multiplicative":
            readout_in = h
            self.W_d_proj = nn.Linear(cfg.r, h, bias=False)
        else:
            readout_in = cfg.r if cfg.no_base else h + cfg.r
            self.W_d_proj = None
        self.W_out = nn.Linear(readout_in, d, bias=cfg.bias)
        self.register_buffer("grid_lo_buf", torch.tensor(float(cfg.grid_lo)))
        self.register_buffer("grid_hi_buf", torch.tensor(float(cfg.grid_hi)))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        """Initialisation of the reference (``rl_spline_kv_reference.py:252-289``): uniform
        +-sqrt(3/fan_in) for K and W_out, a small lift projection, C zero unless a std is given."""
        cfg = self.cfg
        s_in = (3.0 / cfg.d) ** 0.5
        s_out = (3.0 / self.W_out.in_features) ** 0.5
        nn.init.uniform_(self.K.weight, -s_in, s_in)
        nn.init.uniform_(self.W_out.weight, -s_out, s_out)
        if self.W_d_proj is not None:
            nn.init.uniform_(self.W_d_proj.weight, -0.01, 0.01)
        if cfg.c_init_std > 0:
            nn.init.normal_(self.C, mean=0.0, std=float(cfg.c_init_std))
        elif cfg.init_C_zero:
            with torch.no_grad():
                self.C.zero_()
        else:
            nn.init.normal_(self.C, mean=0.0, std=0.02)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        if x.shape[-1] != cfg.d:
            raise ValueError(f"input last-dim {x.shape[-1]} != d={cfg.d}")
        shape = x.shape
        z = self.K(x.reshape(-1, cfg.d))                                        # [N, h]
        out_dtype, z_full = z.dtype, z
        if self.operator_dtype is not None and z.dtype != self.operator_dtype:
            z = z.to(self.operator_dtype)
        lo, hi, G, lam = float(cfg.grid_lo), float(cfg.grid_hi), int(cfg.G), float(cfg.lambda_scale)
        C = self.C if self.C.dtype == z.dtype else self.C.to(z.dtype)
        if cfg.no_base:
            delta = FlashSplineDelta.apply(z, C, lo, hi, G, lam, cfg.bwd_kernel)              # [N, r]
            y = self.W_out(delta.to(out_dtype))
        elif cfg.gating_mode == "multiplicative":
            delta = FlashSplineDelta.apply(z, C, lo, hi, G, lam, cfg.bwd_kernel)              # [N, r], carries lambda
            y = self.W_out((1.0 + self.W_d_proj(delta.to(out_dtype))) * _phi(z_full, cfg.activation))
        elif (self.fused_readout and cfg.spline_order == 2 and cfg.activation in ("relu_sq", "identity")
              and not torch.is_grad_enabled()):
            y = ops.feature_readout_forward(z, C, self.W_out.weight, lo, hi, G, cfg.activation, lam).to(out_dtype)
            if self.W_out.bias is not None:
                y = y + self.W_out.bias
        elif cfg.spline_order == 1:
            f = SplineFeatureOfOrder.apply(z, C, lo, hi, G, cfg.activation, lam, 1)            # [N, h + r]
            y = self.W_out(f.to(out_dtype))
        else:
            f = FlashSplineFeature.apply(z, C, lo, hi, G, cfg.activation, lam, True, cfg.bwd_kernel,
                                         cfg.fwd_kernel)                                       # [N, h + r]
            y = self.W_out(f.to(out_dtype))
        return y.reshape(shape)

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def extra_repr(self) -> str:
        c = self.cfg
        return (f"d={c.d}, h={self.h} (h_ratio={c.h_ratio}), r={c.r}, G={c.G}, lambda={c.lambda_scale}, "
                f"activation={c.activation}, mode={'no_base' if c.no_base else c.gating_mode}")


__all__ = ["RLSplineKVConfig", "RLSplineKV"]
