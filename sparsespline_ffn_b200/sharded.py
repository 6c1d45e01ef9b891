"""The operator across the GPUs of one node: one process per GPU, ``torch.distributed`` (NCCL
over NVLink) for the only exchange step each mode has.

* Token-sharded (primary): every rank owns a slice of the N tokens and a replica of ``C``.  The
  forward and ``dz`` need no communication; ``dC`` is a sum over tokens, so the float32 partial
  ``dC [h, L, r]`` of every rank is all-reduced and cast to the dtype of ``C`` afterwards.
* Key-sharded: every rank owns ``h / P`` keys (``z[:, slice]``, ``C[slice]``) and all tokens.
  The partial residuals ``lambda * delta [N, r]`` are all-reduced in float32 and rounded once;
  the backward is local because ``g_delta`` is replicated.

The reference has no collective of its own for this operator (its data parallelism lives in an
external training script), so there is no reference interface these replace; they exist so that
the operator's one cross-token and one cross-key reduction are exercised and measured.

The local compute goes through ``_local_forward`` / ``_local_backward`` below (the CUDA library);
tests substitute them to rehearse the collectives with CPU ranks over gloo.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import ops


def token_slice(N: int, world: int, rank: int) -> slice:
    """Contiguous, as-even-as-possible split of N tokens."""
    base, rem = divmod(N, world)
    start = rank * base + min(rank, rem)
    return slice(start, start + base + (1 if rank < rem else 0))


def key_slice(h: int, world: int, rank: int, multiple: int = 8) -> slice:
    """Contiguous split of h keys in units of ``multiple`` keys (the tcgen05 kernels want
    multiples of 8)."""
    units = -(-h // multiple)
    s = token_slice(units, world, rank)
    return slice(min(h, s.start * multiple), min(h, s.stop * multiple))


def _local_forward(z, C, lo, hi, G, activation, lam, with_base, delta_f32):
    return ops.feature_forward(z, C, lo, hi, G, activation, lam, with_base=with_base, delta_f32=delta_f32)


def _local_backward(z, C, go, lo, hi, G, activation, lam, with_base, need_dz, need_dC):
    dz, dC32, _ = ops.feature_backward(z, C, go, lo, hi, G, activation, lam, with_base=with_base,
                                       need_dz=need_dz, need_dC=need_dC, cast_dC=False)
    return dz, dC32


def _world_size(group=None) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def all_reduce_sum_(t: torch.Tensor, group=None) -> torch.Tensor:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


class TokenShardedSplineFeature(torch.autograd.Function):
    """``FlashSplineFeature`` on this rank's tokens; ``dC`` summed over the ranks of ``group``."""

    @staticmethod
    def forward(ctx, z, C, grid_lo, grid_hi, G, activation, lambda_scale, group=None):
        f = _local_forward(z.detach(), C.detach(), grid_lo, grid_hi, G, activation, lambda_scale, True, False)
        ctx.save_for_backward(z, C)
        ctx.cfg = (float(grid_lo), float(grid_hi), int(G), activation, float(lambda_scale))
        ctx.group = group
        return f

    @staticmethod
    def backward(ctx, grad_output):
        z, C = ctx.saved_tensors
        lo, hi, G, act, lam = ctx.cfg
        need_dz, need_dC = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if need_dz and need_dC and _world_size(ctx.group) > 1:
            # dC first, its all-reduce started asynchronously, then dz while the exchange is in flight
            # (the second call repeats the small gradient-packing kernels: about 20 us for a 100 us overlap)
            _, dC32 = _local_backward(z.detach(), C.detach(), grad_output, lo, hi, G, act, lam, True, False, True)
            work = dist.all_reduce(dC32, op=dist.ReduceOp.SUM, group=ctx.group, async_op=True)
            dz, _ = _local_backward(z.detach(), C.detach(), grad_output, lo, hi, G, act, lam, True, True, False)
            work.wait()
            return dz, dC32.to(C.dtype), None, None, None, None, None, None
        dz, dC32 = _local_backward(z.detach(), C.detach(), grad_output, lo, hi, G, act, lam, True, need_dz, need_dC)
        dC = None
        if need_dC:
            dC = all_reduce_sum_(dC32, ctx.group).to(C.dtype)
        return dz, dC, None, None, None, None, None, None


def token_sharded_spline_feature(z_local, C, grid_lo=-3.0, grid_hi=3.0, G=20, activation="relu_sq",
                                 lambda_scale=1.0, group=None):
    return TokenShardedSplineFeature.apply(z_local, C, grid_lo, grid_hi, G, activation, lambda_scale, group)


class KeyShardedSplineFeature(torch.autograd.Function):
    """This rank's key slice: returns ``(phi(z_local) [N, h_local], lambda*delta [N, r])`` where the
    residual is the sum over all ranks' keys (all-reduced in float32, rounded once)."""

    @staticmethod
    def forward(ctx, z_local, C_local, grid_lo, grid_hi, G, activation, lambda_scale, group=None):
        act, delta32 = _local_forward(z_local.detach(), C_local.detach(), grid_lo, grid_hi, G, activation,
                                      lambda_scale, True, True)
        delta = all_reduce_sum_(delta32, group).to(z_local.dtype)
        ctx.save_for_backward(z_local, C_local)
        ctx.cfg = (float(grid_lo), float(grid_hi), int(G), activation, float(lambda_scale))
        return act, delta

    @staticmethod
    def backward(ctx, g_act, g_delta):
        z, C = ctx.saved_tensors
        lo, hi, G, act, lam = ctx.cfg
        need_dz, need_dC = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        # the two halves go to the library with their own pointers and strides (no [N, h+r] copy)
        dz, dC32 = _local_backward(z.detach(), C.detach(), (g_act, g_delta), lo, hi, G, act, lam, True, need_dz,
                                   need_dC)
        dC = dC32.to(C.dtype) if need_dC else None
        return dz, dC, None, None, None, None, None, None


def key_sharded_spline_feature(z_local, C_local, grid_lo=-3.0, grid_hi=3.0, G=20, activation="relu_sq",
                               lambda_scale=1.0, group=None):
    return KeyShardedSplineFeature.apply(z_local, C_local, grid_lo, grid_hi, G, activation, lambda_scale, group)
