"""Multi-GPU use of the KDA path: one process per GPU.

* (batch, head) sharding -- ``shard_ranges``: every (sequence, head) pair is an independent
  recurrence, so ranks work on disjoint shards with no collective.
* context parallelism for one long sequence -- ``cp_chunk_forward``: rank r owns a contiguous
  slice of whole 64-token chunks.  A slice maps its entering state affinely to its leaving state,
  ``h_out = M_r h_in + b_r`` with a dense [K, K] transition per head, so only the fp32 boundary
  state [H, K, V] travels, along a point-to-point prefix chain (NCCL send/recv over NVLink):

      1. every rank, in parallel: the chunk-parallel part of its slice (pairwise products, solve,
         w, u, kg, qg); middle ranks also run the recurrence from a zero state (-> b_r) and from an
         identity state with u = 0 (-> M_r);
      2. chain: recv h_in from rank r-1, h_out = M_r h_in + b_r, send to rank r+1 (the first rank
         sends its true leaving state, the last rank only receives);
      3. every rank, in parallel: the recurrence with the true h_in -> outputs.

The reference has no multi-GPU code on this path (docs/linear.md:220-222 leaves context
parallelism to the caller); the per-slice math is the chunk recurrence of
attn_gym/linear/kda/naive.py:99-138 applied to an identity initial state.
"""

from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch


def shard_ranges(batch: int, heads: int, world: int, rank: int) -> Tuple[slice, slice]:
    """Split (batch, head) work over ``world`` ranks: batch first, then heads.

    Returns (batch slice, head slice) of this rank; together the ranks tile the grid exactly.
    """
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if batch % world == 0:
        per = batch // world
        return slice(rank * per, (rank + 1) * per), slice(0, heads)
    if world % batch == 0 and heads % (world // batch) == 0:
        split = world // batch
        per = heads // split
        b, h = divmod(rank, split)
        return slice(b, b + 1), slice(h * per, (h + 1) * per)
    if heads % world == 0:
        per = heads // world
        return slice(0, batch), slice(rank * per, (rank + 1) * per)
    raise ValueError(f"cannot tile batch={batch} x heads={heads} over {world} ranks")


class CudaSlice:
    """One rank's slice on the CUDA kernels: ``prepare`` once, then any number of state passes."""

    def __init__(self, q, k, v, gate, beta):
        from . import _cabi
        from .ops import _dense_offsets

        self._cabi = _cabi
        batch, tokens, heads, _ = q.shape
        self.shape = (batch, tokens, heads)
        q, k, v = (t.to(torch.bfloat16).contiguous() for t in (q, k, v))
        self.gate, beta = gate.float().contiguous(), beta.float().contiguous()
        self.cu, self.offsets, capacity = _dense_offsets(q)
        self.like_v = v
        self.aqk = torch.empty(batch, tokens, heads, 64, dtype=q.dtype, device=q.device)
        akk = torch.empty_like(self.aqk)
        nbytes = _cabi.lib().kda_chunk_fwd_workspace_bytes(batch * tokens, heads)
        self.ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
        _cabi.call("kda_chunk_fwd_prepare", 2, _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v),
                   _cabi.ptr(self.gate), _cabi.ptr(beta), _cabi.ptr(self.aqk), _cabi.ptr(akk),
                   _cabi.ptr(self.cu), _cabi.ptr(self.offsets), batch, batch * tokens, heads,
                   capacity, _cabi.ptr(self.ws), nbytes, _cabi.stream())

    def _state(self, h_in, want_out, use_u):
        c = self._cabi
        batch, tokens, heads = self.shape
        out = torch.empty_like(self.like_v) if want_out else None
        final = torch.empty(batch, heads, 128, 128, dtype=torch.float32, device=self.gate.device)
        h_in = None if h_in is None else h_in.float().contiguous()
        c.call("kda_chunk_fwd_state", 1, c.ptr(self.gate), c.ptr(h_in), c.ptr(final), c.ptr(out),
               c.ptr(self.aqk), c.ptr(self.cu), c.ptr(self.offsets), batch, batch * tokens, heads,
               c.ptr(self.ws), int(use_u), c.stream())
        return out, final

    def run(self, h_in):
        """(outputs, leaving state) for the entering state ``h_in`` (None = zeros)."""
        return self._state(h_in, True, True)

    def zero_state_result(self):
        """b: the leaving state for a zero entering state."""
        return self._state(None, False, True)[1]

    def transition(self):
        """M [B, H, K, K]: the leaving state of the homogeneous recurrence started at identity."""
        batch, _, heads = self.shape
        eye = torch.eye(128, device=self.gate.device).expand(batch, heads, 128, 128).contiguous()
        return self._state(eye, False, False)[1]

    def affine(self, trans, h_in, b):
        c = self._cabi
        out = torch.empty_like(b)
        c.call("kda_state_affine", 1, c.ptr(trans.contiguous()), c.ptr(h_in.contiguous()),
               c.ptr(b.contiguous()), c.ptr(out), b.shape[0] * b.shape[1], b.shape[2], b.shape[3],
               c.stream())
        return out


def cp_chunk_forward(q, k, v, cumulative_gate, beta, initial_state=None, *, group=None,
                     slice_factory: Callable = CudaSlice, rank: Optional[int] = None,
                     world: Optional[int] = None, send: Optional[Callable] = None,
                     recv: Optional[Callable] = None):
    """Context-parallel chunked forward of this rank's slice ``[1, T_local, H, 128]``.

    ``T_local`` must be a multiple of 64 on every rank but the last, so that slices hold whole
    chunks and the chunk-local cumulative gate needs no exchange.  ``initial_state`` is used on rank
    0 only.  Returns (local output, state leaving this slice); on the last rank the second result is
    the final state of the whole sequence.  Only boundary states are communicated:
    ``send(tensor, dst)`` / ``recv(tensor, src)`` default to torch.distributed point-to-point calls.
    """
    if rank is None:
        import torch.distributed as dist

        rank, world = dist.get_rank(group), dist.get_world_size(group)
    if send is None:
        import torch.distributed as dist

        def send(t, dst):
            dist.send(t, dst, group=group)

        def recv(t, src):
            dist.recv(t, src, group=group)

    last = rank + 1 == world
    if not last and q.shape[1] % 64:
        raise ValueError("every slice but the last must hold whole 64-token chunks")
    part = slice_factory(q, k, v, cumulative_gate, beta)           # step 1, all ranks in parallel
    if rank == 0:
        out, h_out = part.run(initial_state)
        if not last:
            send(h_out, 1)
        return out, h_out
    b = trans = None
    if not last:                                                   # still step 1
        b, trans = part.zero_state_result(), part.transition()
    h_in = torch.empty(q.shape[0], q.shape[2], q.shape[3], v.shape[-1], dtype=torch.float32,
                       device=q.device)
    recv(h_in, rank - 1)                                           # step 2
    if not last:
        send(part.affine(trans, h_in, b), rank + 1)
    return part.run(h_in)                                          # step 3


__all__ = ["shard_ranges", "cp_chunk_forward", "CudaSlice"]
