"""Routing metadata for sequence-relative 64-token chunks in a packed token buffer.

Mirrors attn_gym/linear/kda/chunk_schedule.py:49-137.  ``chunk_offsets`` is the exclusive prefix
sum of per-sequence chunk counts and stays on the device; ``capacity`` is the shape-only upper
bound on active chunks that sizes launches and workspaces, so nothing here reads device memory
on the host.
"""

from __future__ import annotations

from typing import NamedTuple

import torch


class RaggedChunkMetadata(NamedTuple):
    cu_seqlens: torch.Tensor
    chunk_offsets: torch.Tensor
    capacity: int
    chunk_size: int

    def validate_chunk_size(self, chunk_size: int) -> None:
        if self.chunk_size != chunk_size:
            raise ValueError(
                f"metadata chunk size must match chunk_size={chunk_size}, got {self.chunk_size}")


def chunk_capacity(tokens: int, num_sequences: int, chunk_size: int) -> int:
    """Largest number of chunks any boundary placement can produce (chunk_schedule.py:101-118)."""
    if tokens < 0:
        raise ValueError(f"tokens must be nonnegative, got {tokens}")
    if num_sequences < 1:
        raise ValueError(f"num_sequences must be positive, got {num_sequences}")
    if chunk_size < 1:
        raise ValueError(f"chunk_size must be positive, got {chunk_size}")
    nonempty = min(tokens, num_sequences)
    if nonempty == 0:
        return 0
    return nonempty + (tokens - nonempty) // chunk_size


def prepare_ragged_chunk_metadata(cu_seqlens: torch.Tensor, tokens: int,
                                  chunk_size: int) -> RaggedChunkMetadata:
    if cu_seqlens.ndim != 1 or cu_seqlens.shape[0] < 2:
        raise ValueError("cu_seqlens must have shape [num_sequences + 1]")
    if cu_seqlens.dtype not in (torch.int32, torch.int64) or not cu_seqlens.is_contiguous():
        raise ValueError("cu_seqlens must be contiguous int32")
    if not cu_seqlens.is_cuda:
        raise ValueError("cu_seqlens must be a CUDA tensor")
    if cu_seqlens.dtype == torch.int64:
        cu_seqlens = cu_seqlens.to(torch.int32)
    capacity = chunk_capacity(tokens, cu_seqlens.shape[0] - 1, chunk_size)
    offsets = torch.ops.kda_b200.kda_prepare_chunk_offsets(cu_seqlens, tokens, chunk_size)
    return RaggedChunkMetadata(cu_seqlens, offsets, capacity, chunk_size)


def dense_metadata(batch: int, tokens: int, chunk_size: int, device) -> RaggedChunkMetadata:
    """The packed description of a dense [batch, tokens] input: equal-length sequences."""
    per_row = (tokens + chunk_size - 1) // chunk_size
    steps = torch.arange(batch + 1, dtype=torch.int32, device=device)
    return RaggedChunkMetadata(steps * tokens, steps * per_row, batch * per_row, chunk_size)


__all__ = ["RaggedChunkMetadata", "chunk_capacity", "prepare_ragged_chunk_metadata",
           "dense_metadata"]
