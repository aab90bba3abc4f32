"""``KDAAttention``: the trainable KDA layer assembled from this package's kernels.

Same module interface as the reference's example layer (examples/kda_training.py:151-538):
constructor arguments, parameter names and shapes, the ``forward`` signature and the
``KDAAttentionOutput`` result, so a checkpoint or a caller of that module fits this one.  Data
flow of ``forward`` (reference lines in brackets):

    hidden --qkv_proj--> qkv --causal_conv1d + SiLU--> q | k | v           [:358-410]
    q, k --l2norm--> unit rows                                             [:412-421]
    hidden --f_a_proj, f_b_proj--> raw gate;  hidden --beta_proj, sigmoid--> beta   [:423-446]
    raw gate --bounded_gate_cumsum--> cumulative log2 gate                 [:448-475]
    chunk_kda(q, k, v, gate, beta) --> o, final state                      [:477-505]
    o, g_b_proj(g_a_proj(hidden)) --gated_output_norm--> y --out_proj--> result    [:507-539]

The projections are cuBLAS GEMMs (``F.linear``); everything between them is this package:
one conv kernel, one gate kernel, the chunked core with the q / k L2 normalisation fused into its
first forward and last backward kernel (``fuse_qk_norm=False`` runs the two l2norm launches of the
reference instead), and the output epilogue ``rms_norm(o) * weight * sigmoid(gate logits)`` as ONE
kernel where the reference runs three.
Packed inputs share one chunk schedule between the gate and the core, as in the reference.
``backend="reference"`` evaluates the same layer in eager fp32 PyTorch (dense inputs only), for
parity checks; there is no fallback from one backend to the other.
"""

from __future__ import annotations

import math
from typing import NamedTuple, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .chunk_schedule import prepare_ragged_chunk_metadata
from .fused import chunk_forward as _chunk_kda
from .masking import active_token_mask, mask_inactive_token_gradients, mask_inactive_tokens
from .preops import _bounded_gate_cumsum, causal_conv1d, gated_output_norm, l2norm
from .reference_impl import reference_kda

_LOG2E = math.log2(math.e)


class KDAAttentionOutput(NamedTuple):
    """Hidden states and optional recurrent and convolution states."""

    hidden_states: torch.Tensor
    final_state: Optional[torch.Tensor]
    final_conv_state: Optional[torch.Tensor]


class KDAAttention(nn.Module):
    """KDA attention layer.  ``mask_inactive_capacity=True`` makes a packed input whose buffer is
    longer than ``cu_seqlens[-1]`` safe for training: the rows past the end are zeroed on the way in
    and kept out of every weight gradient (the primitives leave them undefined)."""

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, *, chunk_size: int = 64,
                 short_conv_kernel_size: int = 4, lower_bound: float = -5.0,
                 backend: str = "fused", fastmath: bool = False, rms_norm_eps: float = 1e-5,
                 compute_dtype: Optional[torch.dtype] = None, device=None,
                 mask_inactive_capacity: bool = False, fuse_qk_norm: bool = True) -> None:
        super().__init__()
        if hidden_size < 1 or num_heads < 1 or head_dim < 1:
            raise ValueError("hidden_size, num_heads, and head_dim must be positive")
        if chunk_size < 1:
            raise ValueError(f"chunk_size must be positive, got {chunk_size}")
        if short_conv_kernel_size < 1:
            raise ValueError(f"short_conv_kernel_size must be positive, got {short_conv_kernel_size}")
        if not math.isfinite(lower_bound) or lower_bound > 0:
            raise ValueError(f"lower_bound must be finite and non-positive, got {lower_bound}")
        if backend not in ("reference", "fused"):
            raise ValueError(f"backend must be 'reference' or 'fused', got {backend!r}")
        if backend == "fused" and (head_dim != 128 or chunk_size != 64):
            raise ValueError("the fused backend requires head_dim=128 and chunk_size=64")
        self.hidden_size, self.num_heads, self.head_dim = hidden_size, num_heads, head_dim
        self.chunk_size, self.lower_bound, self.backend = chunk_size, lower_bound, backend
        self.fastmath, self.rms_norm_eps = fastmath, rms_norm_eps
        self.mask_inactive_capacity = mask_inactive_capacity
        self.fuse_qk_norm = fuse_qk_norm
        self.compute_dtype = ((torch.bfloat16 if backend == "fused" else torch.float32)
                              if compute_dtype is None else compute_dtype)
        if backend == "fused" and self.compute_dtype != torch.bfloat16:
            raise ValueError("the fused backend requires compute_dtype=torch.bfloat16")
        width = num_heads * head_dim
        kw = {"device": device}
        self.qkv_proj = nn.Linear(hidden_size, 3 * width, bias=False, **kw)
        self.qkv_conv1d = nn.Conv1d(3 * width, 3 * width, short_conv_kernel_size, groups=3 * width,
                                    bias=False, **kw)
        self.beta_proj = nn.Linear(hidden_size, num_heads, bias=False, **kw)
        self.f_a_proj = nn.Linear(hidden_size, head_dim, bias=False, **kw)
        self.f_b_proj = nn.Linear(head_dim, width, bias=False, **kw)
        self.g_a_proj = nn.Linear(hidden_size, head_dim, bias=False, **kw)
        self.g_b_proj = nn.Linear(head_dim, width, bias=False, **kw)
        self.output_norm_weight = nn.Parameter(torch.ones(head_dim, device=device, dtype=torch.float32))
        self.out_proj = nn.Linear(width, hidden_size, bias=False, **kw)
        self.A_log = nn.Parameter(torch.zeros(num_heads, device=device, dtype=torch.float32))
        self.dt_bias = nn.Parameter(torch.zeros(num_heads, head_dim, device=device, dtype=torch.float32))

    # ---- stages -------------------------------------------------------------------------------
    def _linear(self, x, layer):
        return F.linear(x, layer.weight.to(self.compute_dtype))

    def short_convolution(self, qkv, initial_state, *, cu_seqlens=None, return_final_state=False):
        batch, tokens, channels = qkv.shape
        hist = self.qkv_conv1d.kernel_size[0] - 1
        nseq = batch if cu_seqlens is None else cu_seqlens.shape[0] - 1
        if initial_state is not None:
            if tuple(initial_state.shape) != (nseq, hist, channels):
                raise ValueError(f"initial_conv_state must have shape {(nseq, hist, channels)}, "
                                 f"got {tuple(initial_state.shape)}")
            initial_state = initial_state.to(device=qkv.device, dtype=qkv.dtype).contiguous()
        weight = self.qkv_conv1d.weight[:, 0].to(self.compute_dtype)
        if self.backend == "fused":
            result = causal_conv1d(qkv, weight, activation="silu", initial_state=initial_state,
                                   cu_seqlens=cu_seqlens, return_final_state=return_final_state)
            return result if return_final_state else (result, None)
        if initial_state is None:
            initial_state = qkv.new_zeros(nseq, hist, channels)
        ext = torch.cat((initial_state, qkv), 1)
        out = F.silu(F.conv1d(ext.transpose(1, 2), self.qkv_conv1d.weight.to(self.compute_dtype),
                              groups=channels).transpose(1, 2))
        return out, (ext[:, tokens:].clone() if return_final_state else None)

    def gate_projections(self, hidden):
        batch, tokens, _ = hidden.shape
        raw = self._linear(self._linear(hidden, self.f_a_proj), self.f_b_proj)
        beta = self._linear(hidden, self.beta_proj).view(batch, tokens, self.num_heads).float().sigmoid()
        return raw.view(batch, tokens, self.num_heads, self.head_dim).contiguous(), beta

    def _reference_core(self, q, k, v, raw_gate, beta, initial_state, return_final_state):
        """Eager fp32 evaluation of the normalisation, the gate and the recurrence (dense input)."""
        q, k, v = q.float(), k.float(), v.float()
        q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6)
        k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        z = raw_gate.float() + self.dt_bias
        gate = self.lower_bound * torch.sigmoid(self.A_log.exp().view(1, 1, -1, 1) * z) * _LOG2E
        batch, tokens = gate.shape[:2]
        pad = (-tokens) % self.chunk_size
        cum = F.pad(gate, (0, 0, 0, 0, 0, pad)).view(batch, -1, self.chunk_size, *gate.shape[2:])
        cum = cum.cumsum(2).view(batch, -1, *gate.shape[2:])[:, :tokens]
        return reference_kda("chunk", q, k, v, cum, beta, initial_state, None, return_final_state)

    # ---- forward ------------------------------------------------------------------------------
    def forward(self, hidden_states, initial_state=None, *, initial_conv_state=None, cu_seqlens=None,
                return_final_state: bool = False) -> KDAAttentionOutput:
        """hidden_states ``[B, T, hidden]`` (packed: ``[1, T, hidden]`` with ``cu_seqlens``);
        ``initial_state [N, H, D, D]``; ``initial_conv_state [N, W - 1, 3 H D]``."""
        if hidden_states.ndim != 3 or hidden_states.shape[-1] != self.hidden_size:
            raise ValueError(f"hidden_states must have shape [B, T, {self.hidden_size}], "
                             f"got {tuple(hidden_states.shape)}")
        batch, tokens, _ = hidden_states.shape
        if batch == 0 or tokens == 0:
            raise ValueError("batch size and sequence length must be greater than zero")
        if cu_seqlens is not None and self.backend != "fused":
            raise ValueError("packed cu_seqlens currently require backend='fused'")
        nseq = batch if cu_seqlens is None else cu_seqlens.shape[0] - 1
        if initial_state is not None:
            expect = (nseq, self.num_heads, self.head_dim, self.head_dim)
            if tuple(initial_state.shape) != expect:
                raise ValueError(f"initial_state must have shape {expect}, got {tuple(initial_state.shape)}")
            initial_state = initial_state.to(device=hidden_states.device, dtype=torch.float32)
        mask = (active_token_mask(hidden_states, cu_seqlens)
                if self.mask_inactive_capacity and cu_seqlens is not None else None)
        hidden = mask_inactive_tokens(hidden_states, mask).to(self.compute_dtype)
        qkv = mask_inactive_token_gradients(self._linear(hidden, self.qkv_proj), mask)
        qkv, final_conv_state = self.short_convolution(qkv, initial_conv_state, cu_seqlens=cu_seqlens,
                                                       return_final_state=return_final_state)
        qkv = mask_inactive_tokens(qkv, mask)
        q, k, v = qkv.view(batch, tokens, 3, self.num_heads, self.head_dim).unbind(2)
        raw_gate, beta = self.gate_projections(hidden)
        raw_gate = mask_inactive_token_gradients(raw_gate, mask)
        beta = mask_inactive_token_gradients(beta, mask)
        if self.backend == "reference":
            out, final_state = self._reference_core(q, k, v, raw_gate, beta, initial_state,
                                                    return_final_state)
        else:
            if not self.fuse_qk_norm:
                q, k = l2norm(q.contiguous()), l2norm(k.contiguous())
            metadata = (None if cu_seqlens is None
                        else prepare_ragged_chunk_metadata(cu_seqlens, tokens, self.chunk_size))
            gate = _bounded_gate_cumsum(raw_gate, self.A_log, self.dt_bias, chunk_size=self.chunk_size,
                                        lower_bound=self.lower_bound, fastmath=self.fastmath,
                                        metadata=metadata)
            out, final_state = _chunk_kda(q, k, v.contiguous(), gate, beta, initial_state,
                                          metadata=metadata, output_final_state=return_final_state,
                                          fastmath=self.fastmath, normalize_qk=self.fuse_qk_norm)
        out = mask_inactive_tokens(out, mask)
        logits = self._linear(self._linear(hidden, self.g_a_proj), self.g_b_proj).view_as(out)
        if self.backend == "fused":
            gated = gated_output_norm(out, logits, self.output_norm_weight, self.rms_norm_eps)
        else:
            gated = F.rms_norm(out.float(), (self.head_dim,), self.output_norm_weight,
                               eps=self.rms_norm_eps) * logits.float().sigmoid()
        result = self._linear(gated.flatten(-2).to(self.compute_dtype), self.out_proj)
        result = mask_inactive_token_gradients(result, mask)
        return KDAAttentionOutput(result.to(hidden_states.dtype), final_state, final_conv_state)


__all__ = ["KDAAttention", "KDAAttentionOutput"]
