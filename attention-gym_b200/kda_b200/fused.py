"""Autograd wrapper around the fused chunk operators.

Same role and call signature as the reference's ``impl/fused.py`` (chunk_forward :147-216,
_ChunkKDA :35-144): normalise dtypes (q, k, v -> bf16; gate, beta, state -> fp32), pick the
dense or packed operator, save (q, k, v, gate, beta, tape, h0, offsets) and run the first-order
backward operator.  Dense inputs of any batch size and length go to the kernels as equal-length
packed sequences, built inside the operator.

One addition: unless ``recompute=True``, a forward pass that will be differentiated keeps its
intermediates (w, u, kg, qg, v_new and the chunk-entry states, about 1.6 KiB per token and head)
for the backward pass instead of rebuilding them there as the reference does
(bwd/cute/chunk_kda_bwd.py:54-85).  The results are identical; ``recompute=True`` gives the
reference's memory footprint back.
"""

from __future__ import annotations

import torch

from . import ops
from .chunk_schedule import RaggedChunkMetadata, prepare_ragged_chunk_metadata

_CHUNK = 64
_HEAD_DIM = 128


def _validate_fused_constraints(q, v):
    if not q.is_cuda:
        raise ValueError("the fused KDA core requires CUDA tensors")
    if q.shape[-1] != _HEAD_DIM or v.shape[-1] != _HEAD_DIM:
        raise ValueError("the fused KDA core requires K=V=128")


class _ChunkKDA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, gate, beta, initial_state, cu_seqlens, chunk_offsets,
                output_final_state, fastmath, autotune, recompute):
        state = None
        saved = None
        if not recompute and any(ctx.needs_input_grad[:6]):
            out, state, aqk, akk, saved = ops.chunk_fwd_saved_op(
                q, k, v, gate, beta, initial_state, cu_seqlens, chunk_offsets, output_final_state)
        elif cu_seqlens is None:
            if output_final_state:
                out, state, aqk, akk = ops.chunk_fwd_with_state_op(q, k, v, gate, beta,
                                                                   initial_state, autotune)
            else:
                out, aqk, akk = ops.chunk_fwd_op(q, k, v, gate, beta, initial_state, autotune)
        elif output_final_state:
            out, state, aqk, akk = ops.chunk_fwd_ragged_with_state_op(
                q, k, v, gate, beta, initial_state, cu_seqlens, chunk_offsets, autotune)
        else:
            out, aqk, akk = ops.chunk_fwd_ragged_op(q, k, v, gate, beta, initial_state, cu_seqlens,
                                                    chunk_offsets, autotune)
        ctx.save_for_backward(q, k, v, gate, beta, aqk, akk, initial_state, cu_seqlens,
                              chunk_offsets, saved)
        ctx.fastmath, ctx.autotune = fastmath, autotune
        ctx.set_materialize_grads(False)
        return (out, state) if output_final_state else out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, d_output, d_final_state=None):
        (q, k, v, gate, beta, aqk, akk, initial_state, cu_seqlens, chunk_offsets,
         saved) = ctx.saved_tensors
        if saved is not None:
            dq, dk, dv, dg, db, dh0 = ops.chunk_bwd_saved_op(
                q, k, v, gate, beta, aqk, akk, saved, cu_seqlens, chunk_offsets, d_output,
                d_final_state, initial_state, initial_state is not None)
            if initial_state is None:
                dh0 = None
            return dq, dk, dv, dg, db, dh0, None, None, None, None, None, None
        args = (q, k, v, gate, beta, aqk, akk, cu_seqlens, chunk_offsets, d_output, d_final_state,
                initial_state, ctx.fastmath, ctx.autotune)
        if initial_state is not None:
            dq, dk, dv, dg, db, dh0 = ops.chunk_bwd_with_state_grad_op(*args)
        else:
            dq, dk, dv, dg, db = ops.chunk_bwd_op(*args)
            dh0 = None
        return dq, dk, dv, dg, db, dh0, None, None, None, None, None, None


class _ChunkKDAQKNorm(torch.autograd.Function):
    """chunk_kda on unnormalised q and k: the L2 normalisation and its backward run inside the first
    forward kernel and the last backward kernel."""

    @staticmethod
    def forward(ctx, q, k, v, gate, beta, initial_state, cu_seqlens, chunk_offsets,
                output_final_state, eps):
        keep = any(ctx.needs_input_grad[:6])
        out, state, aqk, akk, saved, rstd_q, rstd_k = ops.chunk_fwd_qknorm_op(
            q, k, v, gate, beta, initial_state, cu_seqlens, chunk_offsets, output_final_state, keep, eps)
        ctx.save_for_backward(q, k, v, gate, beta, aqk, akk, initial_state, cu_seqlens, chunk_offsets,
                              saved, rstd_q, rstd_k)
        ctx.set_materialize_grads(False)
        return (out, state) if output_final_state else out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, d_output, d_final_state=None):
        (q, k, v, gate, beta, aqk, akk, initial_state, cu_seqlens, chunk_offsets, saved, rstd_q,
         rstd_k) = ctx.saved_tensors
        dq, dk, dv, dg, db, dh0 = ops.chunk_bwd_qknorm_op(
            q, k, v, gate, beta, aqk, akk, saved, rstd_q, rstd_k, cu_seqlens, chunk_offsets, d_output,
            d_final_state, initial_state, initial_state is not None)
        return dq, dk, dv, dg, db, (dh0 if initial_state is not None else None), None, None, None, None


def chunk_forward(q, k, v, cumulative_gate, beta, initial_state=None, *, cu_seqlens=None,
                  metadata: RaggedChunkMetadata | None = None, output_final_state=False,
                  fastmath=False, autotune=True, recompute=False, normalize_qk=False,
                  norm_eps=1e-6):
    """Normalise inputs and run the fused chunk operators (reference: impl/fused.py:147-216).
    ``normalize_qk`` fuses ``l2norm(q)``, ``l2norm(k)`` (and their backward) into the core."""
    if metadata is not None:
        assert cu_seqlens is None
        metadata.validate_chunk_size(_CHUNK)
        cu_seqlens = metadata.cu_seqlens
    _validate_fused_constraints(q, v)
    out_dtype, out_shape = q.dtype, q.shape
    q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    cumulative_gate = cumulative_gate.float().contiguous()
    beta = beta.float().contiguous()
    if cu_seqlens is not None and metadata is None:
        metadata = prepare_ragged_chunk_metadata(cu_seqlens, q.shape[1], _CHUNK)
    if initial_state is not None:
        initial_state = initial_state.float().contiguous()
    cu = None if metadata is None else metadata.cu_seqlens
    offsets = None if metadata is None else metadata.chunk_offsets
    if normalize_qk:
        if recompute:
            raise ValueError("normalize_qk keeps the forward intermediates; recompute=True is not available")
        res = _ChunkKDAQKNorm.apply(q, k, v, cumulative_gate, beta, initial_state, cu, offsets,
                                    bool(output_final_state), float(norm_eps))
        out, state = res if output_final_state else (res, None)
    elif output_final_state:
        out, state = _ChunkKDA.apply(q, k, v, cumulative_gate, beta, initial_state, cu, offsets,
                                     True, fastmath, autotune, recompute)
    else:
        out = _ChunkKDA.apply(q, k, v, cumulative_gate, beta, initial_state, cu, offsets, False,
                              fastmath, autotune, recompute)
        state = None
    return out.reshape(out_shape).to(out_dtype), state


__all__ = ["chunk_forward"]
