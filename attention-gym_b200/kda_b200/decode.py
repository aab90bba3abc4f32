"""The decode step as two launches: fused preprocessing, then the paged state update.

``decode_step`` is what a serving layer runs per generated token: the q | k | v projection goes
through the short convolution (paged history, advanced in place) and SiLU, q and k are
L2-normalised, the raw gate projection becomes the bounded per-token log2 gate, and the recurrent
state pool is advanced in place.  The reference exposes these as separate operators
(``causal_conv1d_decode``, ``l2norm``, ``bounded_gate_cumsum(chunk_size=1)``, ``recurrent_kda`` with
``state_indices``) and lists "decode preprocessing and scan are separate launches" as a serving
limitation (attn_gym/linear/kda/api.py:210-212); here the preprocessing is one kernel.
"""

from __future__ import annotations

import torch

from . import ops as _opsmod  # noqa: F401  (registers the operators)
from .api import recurrent_kda
from .preops import MAX_GATE_LOWER_BOUND_MAGNITUDE

_ops = torch.ops.kda_b200


def decode_step(x, conv_weight, conv_state, raw_gate, A_log, dt_bias, beta, state_pool,
                state_indices, *, activation="silu", lower_bound=-5.0, eps=1e-6):
    """One generated token for each of ``N`` sequences.

    x: ``[N, 3 * H * 128]`` (q, then k, then v channels) in bf16 / fp16 / fp32; conv_weight
    ``[3 * H * 128, W]`` and conv_state ``[slots, W - 1, 3 * H * 128]`` in the dtype of x;
    raw_gate ``[N, H, 128]``; A_log ``[H]``; dt_bias ``[H, 128]``; beta ``[N, H]``; state_pool fp32
    ``[slots, H, 128, 128]``.  ``state_indices`` (int32 ``[N]``) selects the slot of both pools for
    each sequence; entries <= 0 are padding (zero output, pools untouched), so slot 0 is never
    used, as in the paged ``recurrent_kda``.  Both pools are advanced in place.  Returns the output ``[N, H, 128]`` in the
    dtype of x.  Inference only.
    """
    if activation not in (None, "silu"):
        raise ValueError(f"unknown activation {activation!r}; built in: None, 'silu'")
    if x.ndim != 2 or conv_weight.ndim != 2 or conv_state.ndim != 3 or state_pool.ndim != 4:
        raise ValueError("expected x [N, C], conv_weight [C, W], conv_state [slots, W-1, C], "
                         "state_pool [slots, H, 128, 128]")
    heads = state_pool.shape[1]
    channels = 3 * heads * 128
    if tuple(state_pool.shape[2:]) != (128, 128) or x.shape[1] != channels:
        raise ValueError("the decode step requires K = V = 128 and x with 3 * H * 128 channels")
    width = conv_weight.shape[1]
    if conv_weight.shape[0] != channels or tuple(conv_state.shape[1:]) != (width - 1, channels):
        raise ValueError("conv_weight must be [C, W] and conv_state [slots, W-1, C]")
    if not 2 <= width <= 8:
        raise ValueError("the decode step requires 2 <= W <= 8")
    if not (x.is_cuda and x.dtype == conv_weight.dtype == conv_state.dtype):
        raise ValueError("x, conv_weight and conv_state must be CUDA tensors of one dtype")
    if tuple(raw_gate.shape) != (x.shape[0], heads, 128) or tuple(beta.shape) != (x.shape[0], heads):
        raise ValueError("raw_gate must be [N, H, 128] and beta [N, H]")
    if not conv_state.is_contiguous() or not state_pool.is_contiguous():
        raise ValueError("the pools must be contiguous: they are advanced in place")
    if state_pool.dtype != torch.float32:
        raise TypeError("the recurrent state pool must use float32")
    if abs(lower_bound) > MAX_GATE_LOWER_BOUND_MAGNITUDE:
        raise ValueError("lower_bound is outside the supported gate range")
    if (state_indices.dtype != torch.int32 or tuple(state_indices.shape) != (x.shape[0],)
            or not state_indices.is_contiguous() or state_indices.device != x.device):
        raise ValueError("state_indices must be a contiguous int32 tensor with one entry per sequence")
    if torch.is_grad_enabled() and any(t.requires_grad for t in (x, conv_weight, raw_gate, beta)):
        raise RuntimeError("decode_step is inference-only and has no backward")
    q, k, v, gate = _ops.kda_decode_prep(x.contiguous(), conv_weight.contiguous(), conv_state,
                                         state_indices, raw_gate, A_log, dt_bias, heads, activation,
                                         float(lower_bound), float(eps))
    out, _ = recurrent_kda(q, k, v, gate, beta.reshape(x.shape[0], 1, heads), state_pool,
                           state_indices=state_indices)
    return out.reshape(x.shape[0], heads, 128)


__all__ = ["decode_step"]
