"""Shared tensor / packed-sequence contract of chunk_kda and recurrent_kda.

Mirrors attn_gym/linear/kda/validation.py:20-72: ValueError for shape, device and packing
violations, TypeError for dtypes.  One deliberate widening: ``cu_seqlens`` may be int32 or
int64 (the reference accepts int32 only); int64 offsets are narrowed to int32 by the caller
after the range check here.
"""

from __future__ import annotations

import torch

SUPPORTED_INPUT_DTYPES = (torch.float16, torch.bfloat16, torch.float32)


def validate_kda_inputs(q, k, v, gate, beta, initial_state, cu_seqlens, *, op_name, gate_name):
    if q.ndim != 4:
        raise ValueError(f"q must have shape [B, T, H, K], got {tuple(q.shape)}")
    batch, tokens, heads, key_dim = q.shape
    if 0 in (batch, tokens, heads, key_dim):
        raise ValueError(f"q must have nonempty dimensions, got {tuple(q.shape)}")
    if k.shape != q.shape:
        raise ValueError(f"k must have shape {tuple(q.shape)}, got {tuple(k.shape)}")
    if gate.shape != q.shape:
        raise ValueError(f"{gate_name} must have shape {tuple(q.shape)}, got {tuple(gate.shape)}")
    if v.ndim != 4 or v.shape[:3] != (batch, tokens, heads) or v.shape[-1] < 1:
        raise ValueError(f"v must have shape [{batch}, {tokens}, {heads}, V], got {tuple(v.shape)}")
    if beta.shape != (batch, tokens, heads):
        raise ValueError(f"beta must have shape {(batch, tokens, heads)}, got {tuple(beta.shape)}")
    if cu_seqlens is not None:
        if batch != 1:
            raise ValueError("packed cu_seqlens require q to have batch size one")
        if cu_seqlens.ndim != 1 or cu_seqlens.shape[0] < 2:
            raise ValueError("cu_seqlens must have shape [num_sequences + 1]")
        if (cu_seqlens.dtype not in (torch.int32, torch.int64) or not cu_seqlens.is_contiguous()
                or cu_seqlens.device != q.device):
            raise ValueError("cu_seqlens must be contiguous int32 (or int64) on q.device")
        if tokens >= 2 ** 31:
            raise ValueError("packed token capacity must fit in int32")
    state_batch = batch if cu_seqlens is None else cu_seqlens.shape[0] - 1
    expected_state = (state_batch, heads, key_dim, v.shape[-1])
    if initial_state is not None and tuple(initial_state.shape) != expected_state:
        raise ValueError(
            f"initial_state must have shape {expected_state}, got {tuple(initial_state.shape)}")
    tensors = (q, k, v, gate, beta) + (() if initial_state is None else (initial_state,))
    if not all(t.device == q.device for t in tensors):
        raise ValueError(f"all {op_name} inputs must be on the same device")
    if any(t.dtype not in SUPPORTED_INPUT_DTYPES for t in tensors):
        names = ", ".join(str(d) for d in SUPPORTED_INPUT_DTYPES)
        raise TypeError(f"{op_name} inputs must use one of {names}")


__all__ = ["SUPPORTED_INPUT_DTYPES", "validate_kda_inputs"]
