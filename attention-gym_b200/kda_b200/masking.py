"""Inactive-token masking helpers for fixed-capacity packed buffers.

Same three entry points as attn_gym/linear/kda/masking.py:89-150, in their plain
``torch.where`` form (the reference's row kernel is an optimisation outside the KDA hot path).
"""

from __future__ import annotations

import torch


def _check_mask(x, active_mask):
    if x.ndim < 2 or x.shape[0] != 1:
        raise ValueError(f"x must have packed shape [1, T, ...], got {tuple(x.shape)}")
    if tuple(active_mask.shape) != (x.shape[1],):
        raise ValueError(f"active_mask must have shape [{x.shape[1]}], got {tuple(active_mask.shape)}")
    if active_mask.dtype != torch.bool or active_mask.device != x.device:
        raise ValueError(f"active_mask must be torch.bool on {x.device}, got {active_mask.dtype} "
                         f"on {active_mask.device}")


def active_token_mask(x, cu_seqlens):
    """Boolean ``[T]`` predicate of the active packed prefix, ``token < cu_seqlens[-1]``,
    evaluated on the device so a CUDA graph replay follows changing boundaries."""
    if x.ndim < 2 or x.shape[0] != 1:
        raise ValueError(f"x must have packed shape [1, T, ...], got {tuple(x.shape)}")
    if cu_seqlens.ndim != 1 or cu_seqlens.shape[0] < 2:
        raise ValueError("cu_seqlens must have shape [num_sequences + 1]")
    if cu_seqlens.dtype != torch.int32:
        raise ValueError(f"cu_seqlens must have dtype torch.int32, got {cu_seqlens.dtype}")
    if cu_seqlens.device != x.device:
        raise ValueError(f"cu_seqlens must be on the same device as x, got {cu_seqlens.device} "
                         f"and {x.device}")
    if not cu_seqlens.is_contiguous():
        raise ValueError("cu_seqlens must be contiguous")
    return torch.arange(x.shape[1], device=x.device, dtype=torch.int32) < cu_seqlens[-1]


def mask_inactive_tokens(x, active_mask):
    """Zero the values (and therefore the gradients) of inactive token rows."""
    if active_mask is None:
        return x
    _check_mask(x, active_mask)
    return torch.where(active_mask.reshape(1, -1, *((1,) * (x.ndim - 2))), x, 0)


def mask_inactive_token_gradients(x, active_mask):
    """Pass values through unchanged but block gradients of inactive token rows."""
    if active_mask is None:
        return x
    _check_mask(x, active_mask)
    return torch.where(active_mask.reshape(1, -1, *((1,) * (x.ndim - 2))), x, x.detach())


__all__ = ["active_token_mask", "mask_inactive_token_gradients", "mask_inactive_tokens"]
