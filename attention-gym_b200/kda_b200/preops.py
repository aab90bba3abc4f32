"""Bandwidth-bound pre-ops of the KDA layer, behind the reference's Python entry points:
``bounded_gate_cumsum`` (fwd/triton/gate_fwd.py:634-747), ``l2norm`` (fwd/triton/l2norm_fwd.py:231),
``causal_conv1d`` and ``causal_conv1d_decode`` (short_conv/cute.py:3464-3614).
"""

from __future__ import annotations

import math

import torch

from . import ops  # noqa: F401  (registers the operators)
from .chunk_schedule import RaggedChunkMetadata, prepare_ragged_chunk_metadata

_ops = torch.ops.kda_b200

# The intra-chunk gate rebase spans at most 15 tokens of a 16-row block, so one token may decay
# by at most 128 / (15 * log2 e) nats before a rebase factor leaves the fp32 exponent range
# (same limit as the reference, fwd/triton/gate_fwd.py:619-631).
GATE_SPAN_STEPS = 15
MAX_GATE_LOWER_BOUND_MAGNITUDE = 128.0 / (GATE_SPAN_STEPS * math.log2(math.e))


class _BoundedGateCumsum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, raw_gate, A_log, dt_bias, chunk_size, lower_bound, cu_seqlens, chunk_offsets):
        ctx.chunk_size, ctx.lower_bound = chunk_size, lower_bound
        ctx.save_for_backward(raw_gate, A_log, dt_bias, cu_seqlens, chunk_offsets)
        if cu_seqlens is None:
            return _ops.kda_bounded_gate_fwd_dense(raw_gate, A_log, dt_bias, chunk_size,
                                                   lower_bound)
        return _ops.kda_bounded_gate_fwd_ragged(raw_gate, A_log, dt_bias, cu_seqlens,
                                                chunk_offsets, chunk_size, lower_bound)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, d_cumulative):
        raw_gate, A_log, dt_bias, cu_seqlens, chunk_offsets = ctx.saved_tensors
        d_raw, dA, dbias = _ops.kda_bounded_gate_bwd(raw_gate, A_log, dt_bias, d_cumulative,
                                                     cu_seqlens, chunk_offsets, ctx.chunk_size,
                                                     ctx.lower_bound)
        return d_raw, dA, dbias, None, None, None, None


def _bounded_gate_cumsum(raw_gate, A_log, dt_bias, *, chunk_size=64, lower_bound=-5.0,
                         fastmath=False, profile_ranges=False, cu_seqlens=None,
                         metadata: RaggedChunkMetadata | None = None):
    if metadata is not None:
        assert cu_seqlens is None
        metadata.validate_chunk_size(chunk_size)
        cu_seqlens = metadata.cu_seqlens
    if raw_gate.ndim != 4:
        raise ValueError(f"raw_gate must have shape [B, T, H, D], got {tuple(raw_gate.shape)}")
    batch, tokens, heads, dim = raw_gate.shape
    if batch == 0 or tokens == 0 or heads == 0:
        raise ValueError(f"raw_gate must have nonempty B, T, and H, got {tuple(raw_gate.shape)}")
    if dim < 32 or dim > 1024 or dim % 32:
        raise ValueError(
            f"raw_gate head dimension must be a multiple of 32 in [32, 1024], got {dim}")
    if not raw_gate.is_cuda or raw_gate.dtype != torch.bfloat16:
        raise TypeError("bounded_gate_cumsum requires a CUDA bfloat16 raw gate")
    if tuple(A_log.shape) != (heads,) or A_log.dtype != torch.float32:
        raise ValueError(f"A_log must be float32 with shape {(heads,)}, got "
                         f"{tuple(A_log.shape)} and {A_log.dtype}")
    if tuple(dt_bias.shape) != (heads, dim) or dt_bias.dtype != torch.float32:
        raise ValueError(f"dt_bias must be float32 with shape {(heads, dim)}, got "
                         f"{tuple(dt_bias.shape)} and {dt_bias.dtype}")
    if chunk_size <= 0 or chunk_size & (chunk_size - 1):
        raise ValueError(f"chunk_size must be a positive power of two, got {chunk_size}")
    if not -MAX_GATE_LOWER_BOUND_MAGNITUDE <= lower_bound <= 0.0:
        raise ValueError(
            f"lower_bound must lie in [{-MAX_GATE_LOWER_BOUND_MAGNITUDE:.3f}, 0] for the KDA "
            f"intra-chunk gate rebase, got {lower_bound}")
    if not all(t.device == raw_gate.device for t in (A_log, dt_bias)):
        raise ValueError("bounded_gate_cumsum inputs must be on the same device")
    offsets = None
    if cu_seqlens is not None:
        if batch != 1:
            raise ValueError("packed cu_seqlens require raw_gate to have batch size one")
        if cu_seqlens.ndim != 1 or cu_seqlens.shape[0] < 2:
            raise ValueError("cu_seqlens must have shape [num_sequences + 1]")
        if (cu_seqlens.dtype not in (torch.int32, torch.int64)
                or cu_seqlens.device != raw_gate.device or not cu_seqlens.is_contiguous()):
            raise ValueError("cu_seqlens must be contiguous CUDA int32 on raw_gate.device")
        if fastmath:
            raise ValueError("packed bounded_gate_cumsum does not support fastmath=True")
        if metadata is None:
            metadata = prepare_ragged_chunk_metadata(cu_seqlens, tokens, chunk_size)
        cu_seqlens, offsets = metadata.cu_seqlens, metadata.chunk_offsets
    return _BoundedGateCumsum.apply(raw_gate, A_log, dt_bias, chunk_size, float(lower_bound),
                                    cu_seqlens, offsets)


def bounded_gate_cumsum(raw_gate, A_log, dt_bias, *, chunk_size=64, lower_bound=-5.0,
                        fastmath=False, profile_ranges=False, cu_seqlens=None):
    """``log2(e) * chunk_local_cumsum(lower_bound * sigmoid(exp(A_log) * (raw_gate + dt_bias)))``.

    raw_gate: CUDA bf16 ``[B, T, H, D]``; A_log fp32 ``[H]``; dt_bias fp32 ``[H, D]``; returns fp32.
    The prefix sum restarts every ``chunk_size`` tokens and at every packed sequence start.
    Differentiable in raw_gate, A_log and dt_bias.
    """
    return _bounded_gate_cumsum(raw_gate, A_log, dt_bias, chunk_size=chunk_size,
                                lower_bound=lower_bound, fastmath=fastmath,
                                profile_ranges=profile_ranges, cu_seqlens=cu_seqlens)


class _L2Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, eps):
        y, rstd = _ops.kda_l2norm_fwd(x, eps)
        ctx.save_for_backward(y, rstd)
        return y

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dy):
        y, rstd = ctx.saved_tensors
        return _ops.kda_l2norm_bwd(y, rstd, dy), None


def l2norm(x, eps: float = 1e-6, *, cu_seqlens=None):
    """``x * rsqrt(sum(x^2, -1) + eps)`` with fp32 accumulation; rows are independent, so
    ``cu_seqlens`` is accepted for signature compatibility only."""
    if not x.is_cuda:
        raise ValueError("l2norm requires a CUDA tensor")
    if x.shape[-1] % 4:
        raise ValueError("l2norm requires the last dimension to be a multiple of 4")
    return _L2Norm.apply(x, eps)


class _OutputGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o, gate_logits, weight, eps):
        ctx.eps = eps
        ctx.save_for_backward(o, gate_logits, weight)
        return _ops.kda_output_gate_fwd(o, gate_logits, weight, eps)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dy):
        o, gate_logits, weight = ctx.saved_tensors
        d_o, d_logits, d_weight = _ops.kda_output_gate_bwd(o, gate_logits, weight, dy, ctx.eps)
        return d_o, d_logits.to(gate_logits.dtype), d_weight, None


def gated_output_norm(o, gate_logits, weight, eps: float = 1e-5):
    """``rms_norm(o, weight, eps) * sigmoid(gate_logits)`` over the last (head) dimension in one
    pass, fp32 arithmetic, result in ``o.dtype``.

    The epilogue the reference module applies to the output of ``chunk_kda`` as three launches
    (examples/kda_training.py:507-517 ``F.rms_norm``, :519-532 the sigmoid of the gate projection,
    :535-539 their product).  ``o`` and ``gate_logits``: ``[..., D]`` of one shape; ``weight``:
    ``[D]``.  Differentiable in all three.
    """
    if not o.is_cuda:
        raise ValueError("gated_output_norm requires CUDA tensors")
    if o.shape != gate_logits.shape or tuple(weight.shape) != (o.shape[-1],):
        raise ValueError("gate_logits must have the shape of o and weight must be [D]")
    if o.shape[-1] % 4 or o.shape[-1] > 512:
        raise ValueError("gated_output_norm requires the last dimension to be a multiple of 4, at most 512")
    if o.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        raise TypeError("gated_output_norm takes float32, bfloat16 or float16 tensors")
    return _OutputGate.apply(o, gate_logits, weight, float(eps))


class _ShortConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, cu_seqlens, initial_state, activation):
        ctx.activation = activation
        ctx.save_for_backward(x, weight, cu_seqlens, initial_state)
        return _ops.short_conv_fwd(x, weight, cu_seqlens, initial_state, activation=activation)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dy):
        x, weight, cu_seqlens, initial_state = ctx.saved_tensors
        want_state = initial_state is not None and ctx.needs_input_grad[3]
        dx, dw, ds = _ops.short_conv_bwd(x, weight, dy, cu_seqlens, initial_state,
                                         activation=ctx.activation, state_grad=want_state)
        return dx, dw, None, (ds if want_state else None), None


def _validate_conv(x, weight, cu_seqlens, initial_state):
    if x.ndim != 3:
        raise ValueError(f"x must have shape [B, T, C], got {tuple(x.shape)}")
    if not x.is_cuda:
        raise ValueError("causal_conv1d requires CUDA tensors")
    if x.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise TypeError("causal_conv1d supports float16, bfloat16 and float32")
    if weight.ndim != 2 or weight.shape[0] != x.shape[2]:
        raise ValueError(f"weight must have shape [{x.shape[2]}, W], got {tuple(weight.shape)}")
    if weight.dtype != x.dtype or weight.device != x.device:
        raise ValueError("weight must match x in dtype and device")
    if not 1 <= weight.shape[1] <= 8:
        raise ValueError("convolution width must lie in [1, 8]")
    lanes = 16 // x.element_size()
    if x.shape[2] % lanes:
        raise ValueError(f"channels must be a multiple of {lanes} for {x.dtype}")
    nseq = x.shape[0]
    if cu_seqlens is not None:
        if x.shape[0] != 1:
            raise ValueError("packed cu_seqlens require batch size one")
        if (cu_seqlens.ndim != 1 or cu_seqlens.shape[0] < 2 or cu_seqlens.dtype != torch.int32
                or not cu_seqlens.is_contiguous() or cu_seqlens.device != x.device):
            raise ValueError("cu_seqlens must be contiguous CUDA int32 of shape [N + 1]")
        nseq = cu_seqlens.shape[0] - 1
    if initial_state is not None:
        expect = (nseq, weight.shape[1] - 1, x.shape[2])
        if tuple(initial_state.shape) != expect or initial_state.dtype != x.dtype:
            raise ValueError(f"initial_state must have shape {expect} and dtype {x.dtype}")


def _final_conv_state(x, initial_state, width, cu_seqlens):
    """Last ``width - 1`` inputs of every sequence (history shifts in when a sequence is shorter)."""
    hist = width - 1
    b, t, c = x.shape
    if cu_seqlens is None:
        if initial_state is None:
            initial_state = x.new_zeros(b, hist, c)
        return torch.cat((initial_state, x), 1)[:, t:t + hist] if hist else x[:, :0]
    nseq = cu_seqlens.shape[0] - 1
    if initial_state is None:
        initial_state = x.new_zeros(nseq, hist, c)
    starts, ends = cu_seqlens[:-1].long(), cu_seqlens[1:].long()
    offs = torch.arange(hist, device=x.device)
    pos = ends[:, None] - hist + offs[None, :]                 # [nseq, hist] packed positions
    from_input = pos >= starts[:, None]
    gathered = x[0][pos.clamp(0, t - 1)]
    state_pos = (pos - starts[:, None] + hist).clamp(0, max(hist - 1, 0))
    from_state = torch.gather(initial_state, 1, state_pos[:, :, None].expand(-1, -1, c))
    return torch.where(from_input[:, :, None], gathered, from_state)


def causal_conv1d(x, weight, *, activation=None, cu_seqlens=None, initial_state=None,
                  return_final_state=False, forward_config=None, input_grad_config=None,
                  weight_grad_config=None):
    """Causal depthwise convolution ``y[t,c] = act(sum_j w[c,j] x[t-(W-1)+j, c])``.

    x ``[B, T, C]`` (or packed ``[1, T, C]`` with ``cu_seqlens``), weight ``[C, W]``,
    ``initial_state [N, W-1, C]`` oldest first.  ``activation``: None or ``"silu"``.  The
    ``*_config`` arguments of the reference select its tuned schedules; there is one schedule
    here, so they are accepted and ignored.
    """
    if activation not in (None, "silu"):
        raise ValueError(f"unknown activation {activation!r}; built in: None, 'silu'")
    _validate_conv(x, weight, cu_seqlens, initial_state)
    x, weight = x.contiguous(), weight.contiguous()
    if initial_state is not None:
        initial_state = initial_state.contiguous()
    out = _ShortConv.apply(x, weight, cu_seqlens, initial_state, activation)
    if not return_final_state:
        return out
    return out, _final_conv_state(x, initial_state, weight.shape[1], cu_seqlens)


def causal_conv1d_decode(x, weight, state, *, activation=None, state_indices=None,
                         forward_config=None):
    """One token per sequence: x ``[N, C]``, history pool ``state [slots, W-1, C]`` advanced in
    place; ``state_indices`` (int32) selects slots, entries <= 0 give zero output and leave the
    pool untouched.  Inference only."""
    if activation not in (None, "silu"):
        raise ValueError(f"unknown activation {activation!r}; built in: None, 'silu'")
    if x.ndim != 2 or weight.ndim != 2 or state.ndim != 3:
        raise ValueError("expected x [N, C], weight [C, W], state [slots, W-1, C]")
    if weight.shape[1] < 2 or weight.shape[1] > 8:
        raise ValueError("causal_conv1d_decode requires 2 <= W <= 8")
    if tuple(state.shape[1:]) != (weight.shape[1] - 1, x.shape[1]) or weight.shape[0] != x.shape[1]:
        raise ValueError("state must have shape [slots, W-1, C] matching x and weight")
    if not (x.is_cuda and x.dtype == weight.dtype == state.dtype):
        raise ValueError("x, weight and state must be CUDA tensors of one dtype")
    if not state.is_contiguous():
        raise ValueError("state must be contiguous: it is advanced in place")
    if state_indices is not None and (state_indices.dtype != torch.int32
                                      or tuple(state_indices.shape) != (x.shape[0],)):
        raise ValueError("state_indices must be int32 with one entry per sequence")
    if torch.is_grad_enabled() and any(t.requires_grad for t in (x, weight, state)):
        raise RuntimeError("causal_conv1d_decode is inference-only and has no backward")
    return _ops.short_conv_decode(x.contiguous(), weight.contiguous(), state, state_indices,
                                  activation=activation)


__all__ = ["bounded_gate_cumsum", "l2norm", "gated_output_norm", "causal_conv1d", "causal_conv1d_decode",
           "MAX_GATE_LOWER_BOUND_MAGNITUDE"]
