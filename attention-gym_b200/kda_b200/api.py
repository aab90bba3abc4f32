"""Public KDA operations: ``chunk_kda`` (training / prefill) and ``recurrent_kda`` (decode).

Signatures, argument meaning and error behaviour follow attn_gym/linear/kda/api.py:29-247.
``impl="fused"`` runs the sm_100a CUDA kernels of libkda_b200.so; ``impl="reference"`` runs
eager fp32 PyTorch.  Neither ever falls back to the other.

Differences from the reference, all widenings:
  * ``cu_seqlens`` may be int64 as well as int32;
  * ``chunk_kda(impl="fused")`` runs the bf16 chunked kernels for K = V = 128 exactly as the
    reference's fused path does (fp32 q/k/v are rounded to bf16, with or without autograd); fp32
    inference inputs of any other head size up to 256, which the reference's fused path rejects,
    are served by the exact fp32 token scan, and ``exact_fp32=True`` asks for that scan at
    K = V = 128 too.  The scan is serial in T: meant for short sequences and accuracy checks.
"""

from __future__ import annotations

import torch

from .fused import chunk_forward as _fused_chunk_forward
from .ops import recurrent_forward as _fused_recurrent_forward
from .reference_impl import reference_kda
from .types import Impl, resolve_impl
from .validation import validate_kda_inputs


def _narrow_offsets(cu_seqlens):
    if cu_seqlens is not None and cu_seqlens.dtype == torch.int64:
        return cu_seqlens.to(torch.int32)
    return cu_seqlens


def _per_token_gate(cumulative_gate, cu_seqlens):
    """Invert the chunk-local inclusive prefix sum (differences inside each 64-token chunk)."""
    g = cumulative_gate.float()
    tokens = g.shape[1]
    pos = torch.arange(tokens, device=g.device)
    if cu_seqlens is not None:
        start = cu_seqlens.long()
        seq = torch.searchsorted(start, pos, right=True) - 1
        pos = pos - start[seq.clamp(max=start.numel() - 2)]
    first = (pos % 64 == 0)
    prev = torch.cat((torch.zeros_like(g[:, :1]), g[:, :-1]), 1)
    return torch.where(first[None, :, None, None], g, g - prev)


def chunk_kda(q, k, v, cumulative_gate, beta, initial_state=None, *, cu_seqlens=None,
              output_final_state=False, fastmath=False, autotune=True, impl=Impl.FUSED,
              recompute=False, exact_fp32=False, normalize_qk=False, norm_eps=1e-6):
    """Chunk-parallel KDA.

    q, k, cumulative_gate: ``[B, T, H, K]``; v: ``[B, T, H, V]``; beta: ``[B, T, H]``;
    ``cumulative_gate`` is the inclusive log2 decay prefix inside each 64-token chunk (what
    ``bounded_gate_cumsum(chunk_size=64)`` returns); ``initial_state`` has one ``[H, K, V]`` entry
    per logical sequence; ``cu_seqlens [N + 1]`` packs N sequences into a batch-one input (starts
    at 0, non-decreasing, may repeat, may end before T).  Returns ``(output in q.dtype, fp32
    final state or None)``.  ``fastmath`` and ``autotune`` are accepted for signature
    compatibility; there is a single kernel configuration.  ``recompute`` (not in the reference,
    which always behaves as ``True``) makes the backward pass rebuild the forward intermediates
    instead of keeping about 1.6 KiB per token and head between the two passes.  ``exact_fp32``
    (not in the reference; inference only, fp32 inputs) evaluates the recurrence token by token in
    fp32 instead of rounding the operands to bf16.  ``normalize_qk`` (not in the reference, whose
    callers run ``l2norm`` on q and k as separate launches right before this op) takes unnormalised
    q and k and applies ``x * rsqrt(sum(x^2) + norm_eps)`` per row inside the first kernel, and its
    backward inside the last one: the same values as ``chunk_kda(l2norm(q), l2norm(k), ...)`` with
    one full read and write of q and k saved in each direction.
    """
    selected = resolve_impl(impl)
    if selected is Impl.REFERENCE and fastmath:
        raise ValueError("fastmath applies only to impl='fused'")
    validate_kda_inputs(q, k, v, cumulative_gate, beta, initial_state, cu_seqlens,
                        op_name="chunk_kda", gate_name="cumulative_gate")
    cu_seqlens = _narrow_offsets(cu_seqlens)
    if selected is Impl.REFERENCE:
        if normalize_qk:
            qf, kf = q.float(), k.float()
            q = (qf * torch.rsqrt((qf * qf).sum(-1, keepdim=True) + norm_eps)).to(q.dtype)
            k = (kf * torch.rsqrt((kf * kf).sum(-1, keepdim=True) + norm_eps)).to(k.dtype)
        return reference_kda("chunk", q, k, v, cumulative_gate, beta, initial_state, cu_seqlens,
                             output_final_state)
    tensors = (q, k, v, cumulative_gate, beta) + (() if initial_state is None else (initial_state,))
    needs_grad = torch.is_grad_enabled() and any(t.requires_grad for t in tensors)
    off_chunk_shape = q.shape[-1] != 128 or v.shape[-1] != 128
    if exact_fp32 and (needs_grad or q.dtype != torch.float32):
        raise ValueError("exact_fp32 needs float32 q, k, v and no autograd")
    if normalize_qk:
        if exact_fp32:
            raise ValueError("normalize_qk belongs to the chunked bf16 kernels, not to exact_fp32")
        return _fused_chunk_forward(q, k, v, cumulative_gate, beta, initial_state,
                                    cu_seqlens=cu_seqlens, output_final_state=output_final_state,
                                    fastmath=fastmath, autotune=autotune, recompute=recompute,
                                    normalize_qk=True, norm_eps=norm_eps)
    if (q.dtype == torch.float32 and q.is_cuda and not needs_grad and q.shape[-1] <= 256
            and (exact_fp32 or off_chunk_shape)):
        # fp32-accurate path: the token scan on the per-token gate
        gate = _per_token_gate(cumulative_gate, cu_seqlens)
        return _fused_recurrent_forward(q, k, v, gate, beta, initial_state, cu_seqlens=cu_seqlens,
                                        output_final_state=output_final_state)
    return _fused_chunk_forward(q, k, v, cumulative_gate, beta, initial_state,
                                cu_seqlens=cu_seqlens, output_final_state=output_final_state,
                                fastmath=fastmath, autotune=autotune, recompute=recompute)


def _validate_paged_state(q, v, initial_state, cu_seqlens, state_indices, output_final_state):
    if initial_state is None:
        raise ValueError("state_indices requires initial_state as the paged state pool")
    if output_final_state:
        raise ValueError("state_indices advances the pool in place; drop output_final_state")
    if initial_state.ndim != 4 or tuple(initial_state.shape[1:]) != (*q.shape[2:], v.shape[-1]):
        raise ValueError(
            f"the paged state pool must have shape [num_slots, {q.shape[2]}, {q.shape[3]}, "
            f"{v.shape[-1]}], got {tuple(initial_state.shape)}")
    if initial_state.dtype != torch.float32:
        raise TypeError("the paged state pool must use float32")
    if tuple(initial_state.stride()[1:]) != (q.shape[3] * v.shape[-1], v.shape[-1], 1):
        raise TypeError("the paged state pool must be contiguous within each [H, K, V] slot")
    if initial_state.stride(0) < q.shape[2] * q.shape[3] * v.shape[-1]:
        raise ValueError("paged state pool slots must not overlap")
    nseq = q.shape[0] if cu_seqlens is None else cu_seqlens.shape[0] - 1
    if (tuple(state_indices.shape) != (nseq,) or state_indices.dtype != torch.int32
            or not state_indices.is_contiguous() or state_indices.device != q.device):
        raise ValueError(
            f"state_indices must be a contiguous int32 tensor of shape ({nseq},) on q.device, "
            f"got {tuple(state_indices.shape)} of {state_indices.dtype}")


def recurrent_kda(q, k, v, gate, beta, initial_state=None, *, cu_seqlens=None,
                  output_final_state=False, state_indices=None, autotune=True, impl=Impl.FUSED):
    """Token-recurrent KDA for decoding and inference prefill.

    ``gate`` is the *per-token* log2 decay.  With ``state_indices`` (int32, one per sequence)
    ``initial_state`` is a paged pool ``[num_slots, H, K, V]`` advanced in place; entries <= 0 are
    padding (zero output rows, pool untouched).  Inference only.
    """
    selected = resolve_impl(impl)
    validate_kda_inputs(q, k, v, gate, beta, None if state_indices is not None else initial_state,
                        cu_seqlens, op_name="recurrent_kda", gate_name="gate")
    cu_seqlens = _narrow_offsets(cu_seqlens)
    if state_indices is not None:
        _validate_paged_state(q, v, initial_state, cu_seqlens, state_indices, output_final_state)
        if selected is not Impl.FUSED:
            raise ValueError("state_indices requires impl='fused'")
    if selected is Impl.FUSED:
        return _fused_recurrent_forward(q, k, v, gate, beta, initial_state, cu_seqlens=cu_seqlens,
                                        output_final_state=output_final_state,
                                        state_indices=state_indices, autotune=autotune)
    return reference_kda("recurrent", q, k, v, gate, beta, initial_state, cu_seqlens,
                         output_final_state)


__all__ = ["Impl", "chunk_kda", "recurrent_kda"]
