"""Multi-GPU use of the KDA path: one process per GPU.

* (batch, head) sharding -- ``shard_ranges``: every (sequence, head) pair is an independent
  recurrence, so ranks work on disjoint shards with no collective.
* context parallelism for one long sequence -- ``cp_chunk_forward``: rank r owns a contiguous
  slice of whole 64-token chunks.  A slice maps its entering state affinely to its leaving state,
  ``h_out = M_r h_in + b_r`` with a dense [K, K] transition per head, so only the fp32 boundary
  state [H, K, V] travels, along a point-to-point prefix chain (NCCL send/recv over NVLink):

      1. every rank, in parallel: the chunk-parallel part of its slice (pairwise products, solve,
         w, u, kg, qg), then one launch that walks the slice from a zero state (-> b_r and the
         outputs for a zero entering state) and, on other CTAs, from an identity state with u = 0
         (-> M_r, and the number of chunks after which the running transition is exactly zero);
         the first rank runs the plain recurrence with the true initial state instead;
      2. chain: recv h_in from rank r-1, h_out = M_r h_in + b_r, send to rank r+1;
      3. every rank, in parallel: the recurrence with the true h_in over the leading chunks that h_in
         can still reach (all of them if the gates never forget completely), overwriting those
         rows of the step-1 outputs.

The backward pass runs the mirror-image chain (``cp_chunk_backward``): the gradient entering a
slice from the right, ``dh_out``, maps affinely to the one leaving it on the left,
``dh_in = M_r^T dh_out + c_r`` with the same transition ``M_r``; ``c_r`` is the slice's own backward
with ``dh_out = 0``.  So middle ranks compute ``c_r`` in parallel (one forward pass with kept
intermediates, then the reverse state walk alone: ``CudaSliceTape``), the [H, K, V] gradient travels
from the last rank to the first, and every rank then runs its local backward with the true
``dh_out`` from the same intermediates.  ``cp_chunk_kda`` ties both chains into one differentiable call.

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


def _auto_segments(batch, tokens, heads, device):
    """Segments per row for the walks of a slice: as many as fill the SMs, at least 64 chunks each."""
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    chains = batch * heads
    segs = min(8, sms // chains) if chains * 2 <= sms else 1
    return max(1, min(segs, ((tokens + 63) // 64) // 64))


class CudaSlice:
    """One rank's slice on the CUDA kernels: ``prepare`` once, then any number of state passes.

    The rows of the slice are cut into ``segments`` runs of whole chunks (default: as many as fill
    the GPU) that the state kernels walk in parallel; the affine maps of the segments are composed
    into the map of the slice, and the entering state of every segment follows from the slice's
    entering state by the same maps.  One segment per row is the plain serial walk."""

    def __init__(self, q, k, v, gate, beta, segments=None):
        from . import _cabi

        self._cabi = _cabi
        batch, tokens, heads, _ = q.shape
        dev = q.device
        self.shape = (batch, tokens, heads)
        q, k, v = (t.to(torch.bfloat16).contiguous() for t in (q, k, v))
        self.gate, beta = gate.float().contiguous(), beta.float().contiguous()
        row_chunks = (tokens + 63) // 64
        segs = segments or _auto_segments(batch, tokens, heads, dev)
        seg_chunks = -(-row_chunks // max(1, min(segs, row_chunks)))
        self.segs = -(-row_chunks // seg_chunks)
        self.nseq = batch * self.segs
        idx = torch.arange(self.nseq + 1, dtype=torch.int32, device=dev)
        row, sg = idx // self.segs, idx % self.segs
        chunks = torch.clamp(sg * seg_chunks, max=row_chunks)
        self.cu = (row * tokens + torch.clamp(chunks * 64, max=tokens)).to(torch.int32)
        self.offsets = (row * row_chunks + chunks).to(torch.int32)
        capacity = batch * row_chunks
        self.like_v = v
        self.aqk = torch.empty(batch, tokens, heads, 64, dtype=q.dtype, device=dev)
        akk = torch.empty_like(self.aqk)
        nbytes = _cabi.lib().kda_chunk_fwd_workspace_bytes(batch * tokens, heads)
        self.ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        self._maps = None
        _cabi.call("kda_chunk_fwd_prepare", 2, _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v),
                   _cabi.ptr(self.gate), _cabi.ptr(beta), _cabi.ptr(self.aqk), _cabi.ptr(akk),
                   _cabi.ptr(self.cu), _cabi.ptr(self.offsets), self.nseq, batch * tokens, heads,
                   capacity, _cabi.ptr(self.ws), nbytes, _cabi.stream())

    # ---- single launches over the segments (states are [batch * segments, H, 128, 128]) ----------
    def _state(self, h_in, out, use_u, want_final=True, limit=None):
        c = self._cabi
        batch, tokens, heads = self.shape
        final = (torch.empty(self.nseq, heads, 128, 128, dtype=torch.float32, device=self.gate.device)
                 if want_final else None)
        h_in = None if h_in is None else h_in.float().contiguous()
        c.call("kda_chunk_fwd_state", 1, c.ptr(self.gate), c.ptr(h_in), c.ptr(final), c.ptr(out),
               c.ptr(self.aqk), c.ptr(self.cu), c.ptr(self.offsets), self.nseq, batch * tokens, heads,
               c.ptr(self.ws), int(use_u), c.ptr(limit), c.stream())
        return out, final

    def _segment_maps(self, with_output):
        c = self._cabi
        batch, tokens, heads = self.shape
        dev = self.gate.device
        b = torch.empty(self.nseq, heads, 128, 128, dtype=torch.float32, device=dev)
        trans = torch.empty_like(b)
        out = torch.empty_like(self.like_v) if with_output else None
        limit = torch.zeros(self.nseq, heads, dtype=torch.int32, device=dev)
        c.call("kda_chunk_slice_map", 1, c.ptr(self.gate), c.ptr(b), c.ptr(trans), c.ptr(out),
               c.ptr(limit), c.ptr(self.aqk), c.ptr(self.cu), c.ptr(self.offsets), self.nseq,
               batch * tokens, heads, c.ptr(self.ws), c.stream())
        return out, b, trans, limit

    def _by_segment(self, t):
        batch, _, heads = self.shape
        return t.view(batch, self.segs, heads, 128, 128)

    def affine(self, trans, h_in, b):
        """trans @ h_in + b for stacks of [.., 128, 128] fp32 matrices."""
        c = self._cabi
        out = torch.empty_like(b)
        trans, h_in, b = trans.contiguous(), h_in.contiguous(), b.contiguous()
        c.call("kda_state_affine", 1, c.ptr(trans), c.ptr(h_in), c.ptr(b), c.ptr(out),
               b.numel() // (128 * 128), 128, 128, c.stream())
        return out

    # ---- the slice as a whole (states are [batch, H, 128, 128]) ----------------------------------
    def slice_map(self, with_output=True):
        """Everything that does not depend on the entering state, in one launch plus a few tiny
        compositions: (outputs for zero entering states or None, b, M, chunk limits) with
        ``leaving state = M @ entering state + b`` for the slice.  Half of the CTAs walk the segments
        from zero states, the other half with u = 0 from identity states; the latter stop once the
        running transition is exactly zero and report after how many chunks (int32 per segment and
        head): only those leading chunks of a segment can still feel its entering state."""
        out, b, trans, limit = self._segment_maps(with_output)
        self._maps = (b, trans)
        bs, ms = self._by_segment(b), self._by_segment(trans)
        b_all, m_all = bs[:, 0], ms[:, 0]
        zero = torch.zeros_like(b_all) if self.segs > 1 else None
        for sg in range(1, self.segs):
            b_all = self.affine(ms[:, sg], b_all, bs[:, sg])
            m_all = self.affine(ms[:, sg], m_all, zero)
        return out, b_all.contiguous(), m_all.contiguous(), limit

    def correct(self, out, h_in, limit):
        """Rewrite in ``out`` (outputs for zero entering states) the chunks that the true entering
        state ``h_in`` of the slice can still reach: the first ``limit`` chunks of every segment,
        each walked from its own entering state (the slice's, pushed through the segment maps)."""
        b, trans = self._maps
        bs, ms = self._by_segment(b), self._by_segment(trans)
        batch, _, heads = self.shape
        h_seg = torch.empty(batch, self.segs, heads, 128, 128, dtype=torch.float32, device=out.device)
        h_seg[:, 0] = 0.0 if h_in is None else h_in
        for sg in range(1, self.segs):
            h_seg[:, sg] = self.affine(ms[:, sg - 1], h_seg[:, sg - 1], bs[:, sg - 1])
        self._state(h_seg.view(self.nseq, heads, 128, 128), out, True, want_final=False, limit=limit)
        return out

    def run(self, h_in):
        """(outputs, leaving state) for the entering state ``h_in`` (None = zeros)."""
        if self.segs == 1:
            return self._state(h_in, torch.empty_like(self.like_v), True)
        out, b, trans, limit = self.slice_map()
        h_out = b if h_in is None else self.affine(trans, h_in.float(), b)
        return self.correct(out, h_in, limit), h_out

    def zero_state_result(self):
        """b: the leaving state for a zero entering state (serial walk; one segment only)."""
        assert self.segs == 1
        return self._state(None, None, True)[1]

    def transition(self):
        """M [B, H, K, K]: the leaving state of the homogeneous recurrence started at identity
        (serial walk; one segment only)."""
        assert self.segs == 1
        batch, _, heads = self.shape
        eye = torch.eye(128, device=self.gate.device).expand(batch, heads, 128, 128).contiguous()
        return self._state(eye, None, False)[1]


class ChainTimeout(RuntimeError):
    """A boundary state did not arrive from the neighbouring rank within the host deadline."""


def _cp_forward(q, k, v, cumulative_gate, beta, initial_state=None, *, group=None,
                slice_factory: Callable = CudaSlice, rank: Optional[int] = None,
                world: Optional[int] = None, send: Optional[Callable] = None,
                recv: Optional[Callable] = None, timeout: Optional[float] = None):
    """cp_chunk_forward that also returns the entering state and the slice transition."""
    rank, world, send, recv = _resolve_p2p(group, rank, world, send, recv, timeout)
    last = rank + 1 == world
    if not last and q.shape[1] % 64:
        raise ValueError("every slice but the last must hold whole 64-token chunks")
    part = slice_factory(q, k, v, cumulative_gate, beta)           # step 1, all ranks in parallel
    if rank == 0:
        out, h_out = part.run(initial_state)
        if not last:
            send(h_out, 1)
        return out, h_out, initial_state, None
    out, b, trans, limit = part.slice_map()                        # still step 1
    h_in = torch.empty(q.shape[0], q.shape[2], q.shape[3], v.shape[-1], dtype=torch.float32,
                       device=q.device)
    recv(h_in, rank - 1)                                           # step 2
    h_out = part.affine(trans, h_in, b)
    if not last:
        send(h_out, rank + 1)
    out = part.correct(out, h_in, limit)                           # step 3
    return out, h_out, h_in, trans


def _resolve_p2p(group, rank, world, send, recv, timeout=None):
    """Rank and size inside ``group`` plus send / recv callables that take group-local peer ranks.
    ``timeout`` (seconds) puts a host deadline on every receive: ChainTimeout instead of a rank that
    blocks forever on a neighbour that died."""
    if rank is None:
        import torch.distributed as dist

        rank, world = dist.get_rank(group), dist.get_world_size(group)
    if send is None:
        import datetime
        import time

        import torch.distributed as dist

        def peer(r):      # torch's point-to-point calls take global ranks even with group=
            return r if group is None else dist.get_global_rank(group, r)

        def send(t, dst):
            dist.send(t, peer(dst), group=group)

        def recv(t, src):
            if timeout is None:
                dist.recv(t, peer(src), group=group)
                return
            work = dist.irecv(t, peer(src), group=group)
            failure = f"no boundary state from rank {src} within {timeout} s"
            if dist.get_backend(group) == "gloo":
                # gloo completes a receive only inside wait(); its timed wait closes the pair when
                # it runs out, so the group is good for nothing but tear-down afterwards
                try:
                    work.wait(timeout=datetime.timedelta(seconds=timeout))
                except RuntimeError as exc:
                    raise ChainTimeout(failure) from exc
                return
            deadline = time.monotonic() + timeout      # NCCL: completion is a CUDA event query
            while not work.is_completed():
                if time.monotonic() > deadline:
                    raise ChainTimeout(failure)
                time.sleep(0.0005)
            work.wait()
    return rank, world, send, recv


def cp_chunk_forward(q, k, v, cumulative_gate, beta, initial_state=None, *, group=None,
                     slice_factory: Callable = CudaSlice, rank: Optional[int] = None,
                     world: Optional[int] = None, send: Optional[Callable] = None,
                     recv: Optional[Callable] = None, timeout: Optional[float] = None):
    """Context-parallel chunked forward of this rank's slice ``[1, T_local, H, 128]``.

    ``T_local`` must be a multiple of 64 on every rank but the last, so that slices hold whole
    chunks and the chunk-local cumulative gate needs no exchange.  ``initial_state`` is used on rank
    0 only.  Returns (local output, state leaving this slice); on the last rank the second result is
    the final state of the whole sequence.  Only boundary states are communicated:
    ``send(tensor, dst)`` / ``recv(tensor, src)`` default to torch.distributed point-to-point calls
    inside ``group`` (peer ranks are group-local).  ``timeout`` (seconds) bounds the host's wait for
    the entering state; when it runs out the call raises ``ChainTimeout``.
    """
    return _cp_forward(q, k, v, cumulative_gate, beta, initial_state, group=group,
                       slice_factory=slice_factory, rank=rank, world=world, send=send, recv=recv,
                       timeout=timeout)[:2]


def cuda_slice_grads(q, k, v, cumulative_gate, beta, h_in, d_out, dh_out):
    """Local backward of one slice on the CUDA kernels: the gradients of (output, leaving state)
    with cotangents (d_out, dh_out) with respect to q, k, v, gate, beta and the entering state."""
    from .api import chunk_kda

    batch, heads = q.shape[0], q.shape[2]
    if h_in is None:
        h_in = torch.zeros(batch, heads, q.shape[3], v.shape[3], dtype=torch.float32, device=q.device)
    leaves = [t.detach().requires_grad_() for t in (q, k, v, cumulative_gate, beta, h_in)]
    with torch.enable_grad():
        out, h_out = chunk_kda(*leaves, output_final_state=True)
        return torch.autograd.grad((out, h_out), leaves, (d_out, dh_out))


class CudaSliceTape:
    """One forward pass of a slice with its intermediates kept, for the two backward steps of a middle
    rank: ``state_grad`` (the reverse state walk alone: the gradient of the entering state for a given
    gradient of the leaving one) and ``grads`` (the whole backward pass).  Both read the same tapes;
    neither repeats the forward pass."""

    def __init__(self, q, k, v, cumulative_gate, beta, h_in):
        from . import ops

        batch, heads = q.shape[0], q.shape[2]
        if h_in is None:
            h_in = torch.zeros(batch, heads, q.shape[3], v.shape[3], dtype=torch.float32, device=q.device)
        self.args = (q.to(torch.bfloat16).contiguous(), k.to(torch.bfloat16).contiguous(),
                     v.to(torch.bfloat16).contiguous(), cumulative_gate.float().contiguous(),
                     beta.float().contiguous())
        self.h_in = h_in.float().contiguous()
        self.dtypes = (q.dtype, k.dtype, v.dtype, cumulative_gate.dtype, beta.dtype)
        _, _, self.aqk, self.akk, self.saved = ops.chunk_fwd_saved_op(*self.args, self.h_in, None, None, True)

    def state_grad(self, d_out, dh_out):
        from . import ops

        return ops.chunk_bwd_state_saved_op(self.args[3], self.aqk, self.saved, None, None,
                                            d_out.contiguous(), dh_out)

    def grads(self, d_out, dh_out):
        from . import ops

        dq, dk, dv, dg, db, dh = ops.chunk_bwd_saved_op(*self.args, self.aqk, self.akk, self.saved, None,
                                                        None, d_out.contiguous(), dh_out, self.h_in, True)
        return tuple(t.to(dt) for t, dt in zip((dq, dk, dv, dg, db), self.dtypes)) + (dh,)


def _transposed_affine(trans, dh_out, c):
    """M^T dh_out + c for M [B, H, K, K] and states [B, H, K, V] (fp32)."""
    return torch.baddbmm(c.flatten(0, 1), trans.flatten(0, 1).transpose(1, 2).float(),
                         dh_out.flatten(0, 1).float()).view_as(c)


def cp_chunk_backward(q, k, v, cumulative_gate, beta, h_in, trans, d_out, d_final_state=None, *,
                      group=None, local_grads: Callable = cuda_slice_grads,
                      rank: Optional[int] = None, world: Optional[int] = None,
                      send: Optional[Callable] = None, recv: Optional[Callable] = None):
    """Context-parallel backward of this rank's slice.

    ``h_in`` is the state that entered the slice in the forward chain and ``trans`` the slice
    transition (both as returned by the forward chain; ``trans`` is only needed on middle ranks).
    ``d_out`` is the cotangent of the local output; ``d_final_state`` (last rank only) that of the
    final state.  Returns (dq, dk, dv, d_gate, d_beta, d_h_in); on rank 0 the last one is the
    gradient of the initial state.  Only [B, H, K, V] fp32 state gradients are communicated, from
    rank r + 1 to rank r.
    """
    rank, world, send, recv = _resolve_p2p(group, rank, world, send, recv)
    last = rank + 1 == world
    shape = (q.shape[0], q.shape[2], q.shape[3], v.shape[3])
    if last:
        dh_out = (torch.zeros(shape, dtype=torch.float32, device=q.device)
                  if d_final_state is None else d_final_state.float())
        grads = local_grads(q, k, v, cumulative_gate, beta, h_in, d_out, dh_out)
        if rank > 0:
            send(grads[5].contiguous(), rank - 1)
        return grads
    c = None
    tape = None
    if rank > 0:      # middle rank, in parallel with the others: c = the state gradient for dh_out = 0
        zero = torch.zeros(shape, dtype=torch.float32, device=q.device)
        if local_grads is cuda_slice_grads:
            # one forward pass with kept intermediates serves both steps, and the first step is the
            # reverse state walk alone (no dq, dk, dv, dG, dbeta are formed for the zero cotangent)
            tape = CudaSliceTape(q, k, v, cumulative_gate, beta, h_in)
            c = tape.state_grad(d_out, zero)
        else:
            c = local_grads(q, k, v, cumulative_gate, beta, h_in, d_out, zero)[5]
    dh_out = torch.empty(shape, dtype=torch.float32, device=q.device)
    recv(dh_out, rank + 1)
    if rank > 0:
        send(_transposed_affine(trans, dh_out, c.float()).contiguous(), rank - 1)
    if tape is not None:
        return tape.grads(d_out, dh_out)
    return local_grads(q, k, v, cumulative_gate, beta, h_in, d_out, dh_out)


class _CPChunkKDA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cumulative_gate, beta, initial_state, group):
        out, h_out, h_in, trans = _cp_forward(q, k, v, cumulative_gate, beta, initial_state,
                                              group=group)
        ctx.group = group
        # the initial state is read on rank 0 only; elsewhere it gets no gradient
        ctx.has_h0 = initial_state is not None and _resolve_p2p(group, None, None, None, None)[0] == 0
        ctx.save_for_backward(q, k, v, cumulative_gate, beta, h_in, trans)
        return out, h_out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, d_out, d_h_out):
        q, k, v, gate, beta, h_in, trans = ctx.saved_tensors
        grads = cp_chunk_backward(q, k, v, gate, beta, h_in, trans, d_out.contiguous(), d_h_out,
                                  group=ctx.group)
        dq, dk, dv, dg, db, dh = grads
        return (dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), dg.to(gate.dtype), db.to(beta.dtype),
                dh if ctx.has_h0 else None, None)


def cp_chunk_kda(q, k, v, cumulative_gate, beta, initial_state=None, *, group=None):
    """Differentiable context-parallel ``chunk_kda`` of this rank's slice: the forward boundary-state
    chain and, in backward, the state-gradient chain in the opposite direction.  Returns (local
    output, state leaving the slice).  The cotangent of the leaving state is used on the last rank
    only (on the other ranks it arrives through the chain)."""
    return _CPChunkKDA.apply(q, k, v, cumulative_gate, beta, initial_state, group)


__all__ = ["shard_ranges", "cp_chunk_forward", "cp_chunk_backward", "cp_chunk_kda",
           "cuda_slice_grads", "CudaSlice", "CudaSliceTape", "ChainTimeout"]
