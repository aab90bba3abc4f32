"""torch.library operators of the fused KDA path, bound to the C ABI of libkda_b200.so.

The operator names, argument lists and result arities are those of the reference's private
operators (attn_gym/linear/kda/ops.py:18-136, fwd/triton/gate_fwd.py:379-393,
fwd/triton/l2norm_fwd.py:84,143, bwd/cute/gate_bwd_fused.py:498-502) under the ``kda_b200``
namespace, so the reference can be imported beside this package.  Each CUDA implementation
allocates its outputs and workspace with torch and makes one call into the shared library on
the current stream: no host synchronisation, no second back end, no CPU implementation.
"""

from __future__ import annotations

import torch

from . import _cabi
from .chunk_schedule import chunk_capacity

_CHUNK = 64
_NS = "kda_b200"
_lib = torch.library.Library(_NS, "DEF")


def _define(name, schema):
    _lib.define(f"{name}{schema}")


_FWD = ("(Tensor q, Tensor k, Tensor v, Tensor cumulative_gate, Tensor beta, "
        "Tensor? initial_state, bool autotune)")
_FWD_RAGGED = ("(Tensor q, Tensor k, Tensor v, Tensor cumulative_gate, Tensor beta, "
               "Tensor? initial_state, Tensor cu_seqlens, Tensor chunk_offsets, bool autotune)")
_BWD = ("(Tensor q, Tensor k, Tensor v, Tensor cumulative_gate, Tensor beta, Tensor Aqk, "
        "Tensor Akk, Tensor? cu_seqlens, Tensor? chunk_offsets, Tensor? d_output, "
        "Tensor? d_final_state, {state}, bool fastmath, bool autotune)")
_REC = ("(Tensor q, Tensor k, Tensor v, Tensor gate, Tensor beta, Tensor? initial_state, "
        "Tensor? cu_seqlens, bool autotune)")

_define("kda_chunk_fwd", _FWD + " -> (Tensor, Tensor, Tensor)")
_define("kda_chunk_fwd_with_state", _FWD + " -> (Tensor, Tensor, Tensor, Tensor)")
_define("kda_chunk_fwd_ragged", _FWD_RAGGED + " -> (Tensor, Tensor, Tensor)")
_define("kda_chunk_fwd_ragged_with_state", _FWD_RAGGED + " -> (Tensor, Tensor, Tensor, Tensor)")
_define("kda_chunk_bwd", _BWD.format(state="Tensor? initial_state")
        + " -> (Tensor, Tensor, Tensor, Tensor, Tensor)")
_define("kda_chunk_bwd_with_state_grad", _BWD.format(state="Tensor initial_state")
        + " -> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)")
# Training pair that keeps the forward intermediates instead of rebuilding them in the backward
# pass (no reference counterpart: the reference always recomputes, bwd/cute/chunk_kda_bwd.py:54-85).
# The backward operator also uses the buffer as its workspace (dv2 and dh[c] are written into it),
# hence the mutation annotation.
_define("kda_chunk_fwd_saved",
        "(Tensor q, Tensor k, Tensor v, Tensor cumulative_gate, Tensor beta, Tensor? initial_state, "
        "Tensor? cu_seqlens, Tensor? chunk_offsets, bool want_state) "
        "-> (Tensor, Tensor, Tensor, Tensor, Tensor)")
_define("kda_chunk_bwd_saved",
        "(Tensor q, Tensor k, Tensor v, Tensor cumulative_gate, Tensor beta, Tensor Aqk, Tensor Akk, "
        "Tensor(a!) saved, Tensor? cu_seqlens, Tensor? chunk_offsets, Tensor? d_output, "
        "Tensor? d_final_state, Tensor? initial_state, bool want_state_grad) "
        "-> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)")
# The reverse state-gradient walk of kda_chunk_bwd_saved alone (no reference counterpart: it serves the
# context-parallel backward chain, which needs the gradient of a slice's entering state before the
# state gradient of the next slice has arrived).
_define("kda_chunk_bwd_state_saved",
        "(Tensor cumulative_gate, Tensor Aqk, Tensor(a!) saved, Tensor? cu_seqlens, "
        "Tensor? chunk_offsets, Tensor d_output, Tensor? d_final_state) -> Tensor")
# The chunked pair with the layer's q / k L2 normalisation fused in (no reference counterpart as one
# operator: the reference runs l2norm as separate launches, fwd/triton/l2norm_fwd.py:84,143).
_define("kda_chunk_fwd_qknorm",
        "(Tensor q, Tensor k, Tensor v, Tensor cumulative_gate, Tensor beta, Tensor? initial_state, "
        "Tensor? cu_seqlens, Tensor? chunk_offsets, bool want_state, bool keep, float eps) "
        "-> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)")
_define("kda_chunk_bwd_qknorm",
        "(Tensor q, Tensor k, Tensor v, Tensor cumulative_gate, Tensor beta, Tensor Aqk, Tensor Akk, "
        "Tensor(a!) saved, Tensor rstd_q, Tensor rstd_k, Tensor? cu_seqlens, Tensor? chunk_offsets, "
        "Tensor? d_output, Tensor? d_final_state, Tensor? initial_state, bool want_state_grad) "
        "-> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)")
_define("kda_recurrent_fwd", _REC + " -> (Tensor, Tensor)")
_define("kda_recurrent_fwd_no_state", _REC + " -> Tensor")
_define("kda_recurrent_fwd_paged",
        "(Tensor q, Tensor k, Tensor v, Tensor gate, Tensor beta, Tensor(a!) state_cache, "
        "Tensor state_indices, Tensor? cu_seqlens, bool autotune) -> Tensor")
_define("kda_prepare_chunk_offsets", "(Tensor cu_seqlens, SymInt tokens, int chunk_size) -> Tensor")
_define("kda_bounded_gate_fwd_dense",
        "(Tensor raw_gate, Tensor A_log, Tensor dt_bias, int chunk_size, float lower_bound) -> Tensor")
_define("kda_bounded_gate_fwd_ragged",
        "(Tensor raw_gate, Tensor A_log, Tensor dt_bias, Tensor cu_seqlens, Tensor chunk_offsets, "
        "int chunk_size, float lower_bound) -> Tensor")
_define("kda_bounded_gate_bwd",
        "(Tensor raw_gate, Tensor A_log, Tensor dt_bias, Tensor d_cumulative, Tensor? cu_seqlens, "
        "Tensor? chunk_offsets, int chunk_size, float lower_bound) -> (Tensor, Tensor, Tensor)")
_define("kda_l2norm_fwd", "(Tensor x, float eps) -> (Tensor, Tensor)")
_define("kda_l2norm_bwd", "(Tensor y, Tensor rstd, Tensor dy) -> Tensor")
# output epilogue of the layer (examples/kda_training.py:507-539): RMSNorm * weight * sigmoid(gate)
_define("kda_output_gate_fwd", "(Tensor o, Tensor gate_logits, Tensor weight, float eps) -> Tensor")
_define("kda_output_gate_bwd",
        "(Tensor o, Tensor gate_logits, Tensor weight, Tensor dy, float eps) -> (Tensor, Tensor, Tensor)")
_define("short_conv_fwd",
        "(Tensor x, Tensor weight, Tensor? cu_seqlens=None, Tensor? initial_state=None, *, "
        "str? activation=None) -> Tensor")
_define("short_conv_bwd",
        "(Tensor x, Tensor weight, Tensor grad_output, Tensor? cu_seqlens=None, "
        "Tensor? initial_state=None, *, str? activation=None, bool state_grad=False) "
        "-> (Tensor, Tensor, Tensor)")
_define("short_conv_decode",
        "(Tensor x, Tensor weight, Tensor(a!) state, Tensor? state_indices, *, "
        "str? activation=None) -> Tensor")


# Decode-step preprocessing in one launch (no reference counterpart: the reference runs the conv,
# the two l2norms and the gate as separate launches, kda/api.py:210-212).
_define("kda_decode_prep",
        "(Tensor x, Tensor weight, Tensor(a!) conv_state, Tensor? state_indices, Tensor raw_gate, "
        "Tensor A_log, Tensor dt_bias, int heads, str? activation, float lower_bound, float eps) "
        "-> (Tensor, Tensor, Tensor, Tensor)")


def _require_cuda(t: torch.Tensor, what: str):
    if not t.is_cuda:
        raise ValueError(f"{what} requires CUDA tensors")


# --------------------------------------------------------------------------------------------
# chunked forward / backward
# --------------------------------------------------------------------------------------------
def _dense_offsets(q):
    batch, tokens = q.shape[0], q.shape[1]
    per_row = (tokens + _CHUNK - 1) // _CHUNK
    steps = torch.arange(batch + 1, dtype=torch.int32, device=q.device)
    return steps * tokens, steps * per_row, batch * per_row


def _fwd_workspace_bytes(batch, tokens, heads, packed_nseq, keep):
    """Bytes of the forward workspace (keep: the buffer that is handed on to the backward pass);
    shape-only, so the real and the fake implementations agree."""
    lib = _cabi.lib()
    if packed_nseq is None:
        return int(lib.kda_chunk_fwd_dense_workspace_bytes(batch, tokens, heads, int(keep)))
    if keep:
        return int(lib.kda_chunk_bwd_workspace_bytes(tokens, heads,
                                                     chunk_capacity(tokens, packed_nseq, _CHUNK)))
    return int(lib.kda_chunk_fwd_workspace_bytes(tokens, heads))


def _chunk_fwd_impl(q, k, v, gate, beta, initial_state, cu_seqlens, chunk_offsets, want_state,
                    keep=False):
    _require_cuda(q, "the fused KDA core")
    if q.shape[-1] != 128 or v.shape[-1] != 128:
        raise ValueError("the fused KDA core requires K=V=128")
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise TypeError("the fused KDA core takes bfloat16 q, k, v")
    batch, tokens, heads, _ = q.shape
    packed = cu_seqlens is not None
    if not packed:
        nseq, capacity = batch, None
    else:
        if batch != 1:
            raise ValueError("packed cu_seqlens require batch size one")
        nseq = cu_seqlens.shape[0] - 1
        capacity = chunk_capacity(tokens, nseq, _CHUNK)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    gate = gate.float().contiguous()
    beta = beta.float().contiguous()
    if initial_state is not None:
        initial_state = initial_state.float().contiguous()
    total = batch * tokens
    out = torch.zeros_like(v) if packed else torch.empty_like(v)
    aqk = torch.empty(batch, tokens, heads, _CHUNK, dtype=q.dtype, device=q.device)
    akk = torch.empty_like(aqk)
    state = (torch.empty(nseq, heads, 128, 128, dtype=torch.float32, device=q.device)
             if want_state else None)
    ws_bytes = _fwd_workspace_bytes(batch, tokens, heads, None if not packed else nseq, keep)
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    head = (_cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), _cabi.ptr(gate), _cabi.ptr(beta),
            _cabi.ptr(initial_state), _cabi.ptr(state), _cabi.ptr(out), _cabi.ptr(aqk), _cabi.ptr(akk))
    if packed:
        _cabi.call("kda_chunk_fwd_save" if keep else "kda_chunk_fwd", 3, *head, _cabi.ptr(cu_seqlens),
                   _cabi.ptr(chunk_offsets), nseq, total, heads, 128, 128, capacity,
                   _cabi.ptr(workspace), ws_bytes, _cabi.stream())
    else:
        # dense rows: offsets are built on the device, long rows of small batches are walked in
        # parallel segments
        _cabi.call("kda_chunk_fwd_dense_save" if keep else "kda_chunk_fwd_dense", 3, *head, batch,
                   tokens, heads, 128, 128, _cabi.ptr(workspace), ws_bytes, _cabi.stream())
    if keep:
        return out, state, aqk, akk, workspace
    return out, state, aqk, akk


@torch.library.impl(_lib, "kda_chunk_fwd", "CUDA")
def _chunk_fwd(q, k, v, gate, beta, initial_state, autotune):
    out, _, aqk, akk = _chunk_fwd_impl(q, k, v, gate, beta, initial_state, None, None, False)
    return out, aqk, akk


@torch.library.impl(_lib, "kda_chunk_fwd_with_state", "CUDA")
def _chunk_fwd_with_state(q, k, v, gate, beta, initial_state, autotune):
    return _chunk_fwd_impl(q, k, v, gate, beta, initial_state, None, None, True)


@torch.library.impl(_lib, "kda_chunk_fwd_ragged", "CUDA")
def _chunk_fwd_ragged(q, k, v, gate, beta, initial_state, cu_seqlens, chunk_offsets, autotune):
    out, _, aqk, akk = _chunk_fwd_impl(q, k, v, gate, beta, initial_state, cu_seqlens,
                                       chunk_offsets, False)
    return out, aqk, akk


@torch.library.impl(_lib, "kda_chunk_fwd_ragged_with_state", "CUDA")
def _chunk_fwd_ragged_with_state(q, k, v, gate, beta, initial_state, cu_seqlens, chunk_offsets,
                                 autotune):
    return _chunk_fwd_impl(q, k, v, gate, beta, initial_state, cu_seqlens, chunk_offsets, True)


def _chunk_bwd_impl(q, k, v, gate, beta, aqk, akk, cu_seqlens, chunk_offsets, d_output,
                    d_final_state, initial_state, want_state_grad, saved=None, rstd=None):
    batch, tokens, heads, _ = q.shape
    if cu_seqlens is None:
        cu_seqlens, chunk_offsets, capacity = _dense_offsets(q)
        nseq = batch
        packed = False
    else:
        nseq = cu_seqlens.shape[0] - 1
        capacity = chunk_capacity(tokens, nseq, _CHUNK)
        packed = True
    total = batch * tokens
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    gate = gate.float().contiguous()
    beta = beta.float().contiguous()
    if d_output is None:
        d_output = torch.zeros_like(v)
    d_output = d_output.to(torch.bfloat16).contiguous()
    if d_final_state is not None:
        d_final_state = d_final_state.float().contiguous()
    if initial_state is not None:
        initial_state = initial_state.float().contiguous()
    alloc = torch.zeros_like if packed else torch.empty_like
    dq, dk, dv = alloc(q), alloc(k), alloc(v)
    dg, db = alloc(gate), alloc(beta)
    dh0 = (torch.empty(nseq, heads, 128, 128, dtype=torch.float32, device=q.device)
           if want_state_grad else None)
    ws_bytes = _cabi.lib().kda_chunk_bwd_workspace_bytes(total, heads, capacity)
    if saved is not None:
        if saved.numel() < ws_bytes or saved.dtype != torch.uint8 or not saved.is_cuda:
            raise ValueError("`saved` is not the buffer kda_chunk_fwd_saved returned for these shapes")
        workspace = saved
    else:
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    head = (_cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), _cabi.ptr(gate),
            _cabi.ptr(beta), _cabi.ptr(aqk), _cabi.ptr(akk), _cabi.ptr(initial_state),
            _cabi.ptr(d_output), _cabi.ptr(d_final_state), _cabi.ptr(dq), _cabi.ptr(dk),
            _cabi.ptr(dv), _cabi.ptr(dg), _cabi.ptr(db), _cabi.ptr(dh0), _cabi.ptr(cu_seqlens),
            _cabi.ptr(chunk_offsets), nseq, total, heads, 128, 128, capacity)
    if rstd is not None:
        _cabi.call("kda_chunk_bwd_qknorm_saved", 2, *head, _cabi.ptr(rstd[0]), _cabi.ptr(rstd[1]),
                   _cabi.ptr(workspace), ws_bytes, _cabi.stream())
    else:
        _cabi.call("kda_chunk_bwd_saved" if saved is not None else "kda_chunk_bwd", 5, *head,
                   _cabi.ptr(workspace), ws_bytes, _cabi.stream())
    return dq, dk, dv, dg, db, dh0


@torch.library.impl(_lib, "kda_chunk_bwd", "CUDA")
def _chunk_bwd(q, k, v, gate, beta, aqk, akk, cu_seqlens, chunk_offsets, d_output, d_final_state,
               initial_state, fastmath, autotune):
    return _chunk_bwd_impl(q, k, v, gate, beta, aqk, akk, cu_seqlens, chunk_offsets, d_output,
                           d_final_state, initial_state, False)[:5]


@torch.library.impl(_lib, "kda_chunk_bwd_with_state_grad", "CUDA")
def _chunk_bwd_with_state_grad(q, k, v, gate, beta, aqk, akk, cu_seqlens, chunk_offsets, d_output,
                               d_final_state, initial_state, fastmath, autotune):
    return _chunk_bwd_impl(q, k, v, gate, beta, aqk, akk, cu_seqlens, chunk_offsets, d_output,
                           d_final_state, initial_state, True)


@torch.library.impl(_lib, "kda_chunk_fwd_saved", "CUDA")
def _chunk_fwd_saved(q, k, v, gate, beta, initial_state, cu_seqlens, chunk_offsets, want_state):
    out, state, aqk, akk, saved = _chunk_fwd_impl(q, k, v, gate, beta, initial_state, cu_seqlens,
                                                  chunk_offsets, want_state, keep=True)
    if state is None:
        state = torch.empty(0, dtype=torch.float32, device=q.device)
    return out, state, aqk, akk, saved


@torch.library.impl(_lib, "kda_chunk_bwd_saved", "CUDA")
def _chunk_bwd_saved(q, k, v, gate, beta, aqk, akk, saved, cu_seqlens, chunk_offsets, d_output,
                     d_final_state, initial_state, want_state_grad):
    dq, dk, dv, dg, db, dh0 = _chunk_bwd_impl(q, k, v, gate, beta, aqk, akk, cu_seqlens,
                                              chunk_offsets, d_output, d_final_state, initial_state,
                                              want_state_grad, saved=saved)
    if dh0 is None:
        dh0 = torch.empty(0, dtype=torch.float32, device=q.device)
    return dq, dk, dv, dg, db, dh0


@torch.library.impl(_lib, "kda_chunk_bwd_state_saved", "CUDA")
def _chunk_bwd_state_saved(gate, aqk, saved, cu_seqlens, chunk_offsets, d_output, d_final_state):
    _require_cuda(d_output, "the fused KDA core")
    batch, tokens, heads, dim = d_output.shape
    if dim != 128 or gate.shape[-1] != 128:
        raise ValueError("the fused KDA core requires K=V=128")
    if cu_seqlens is None:
        cu_seqlens, chunk_offsets, capacity = _dense_offsets(d_output)
        nseq = batch
    else:
        nseq = cu_seqlens.shape[0] - 1
        capacity = chunk_capacity(tokens, nseq, _CHUNK)
    total = batch * tokens
    ws_bytes = _cabi.lib().kda_chunk_bwd_workspace_bytes(total, heads, capacity)
    if saved.numel() < ws_bytes or saved.dtype != torch.uint8 or not saved.is_cuda:
        raise ValueError("`saved` is not the buffer kda_chunk_fwd_saved returned for these shapes")
    gate = gate.float().contiguous()
    d_output = d_output.to(torch.bfloat16).contiguous()
    if d_final_state is not None:
        d_final_state = d_final_state.float().contiguous()
    dh0 = torch.empty(nseq, heads, 128, 128, dtype=torch.float32, device=d_output.device)
    _cabi.call("kda_chunk_bwd_state_saved", 1, _cabi.ptr(gate), _cabi.ptr(aqk.contiguous()),
               _cabi.ptr(d_output), _cabi.ptr(d_final_state), _cabi.ptr(dh0), _cabi.ptr(cu_seqlens),
               _cabi.ptr(chunk_offsets), nseq, total, heads, 128, 128, capacity, _cabi.ptr(saved),
               saved.numel(), _cabi.stream())
    return dh0


@torch.library.impl(_lib, "kda_chunk_fwd_qknorm", "CUDA")
def _chunk_fwd_qknorm(q, k, v, gate, beta, initial_state, cu_seqlens, chunk_offsets, want_state, keep,
                      eps):
    _require_cuda(q, "the fused KDA core")
    if q.shape[-1] != 128 or v.shape[-1] != 128:
        raise ValueError("the fused KDA core requires K=V=128")
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise TypeError("the fused KDA core takes bfloat16 q, k, v")
    batch, tokens, heads, _ = q.shape
    packed = cu_seqlens is not None
    if not packed:
        cu_seqlens, chunk_offsets, capacity = _dense_offsets(q)
        nseq = batch
    else:
        if batch != 1:
            raise ValueError("packed cu_seqlens require batch size one")
        nseq = cu_seqlens.shape[0] - 1
        capacity = chunk_capacity(tokens, nseq, _CHUNK)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    gate, beta = gate.float().contiguous(), beta.float().contiguous()
    if initial_state is not None:
        initial_state = initial_state.float().contiguous()
    total = batch * tokens
    out = torch.zeros_like(v) if packed else torch.empty_like(v)
    aqk = torch.empty(batch, tokens, heads, _CHUNK, dtype=q.dtype, device=q.device)
    akk = torch.empty_like(aqk)
    alloc = torch.zeros if packed else torch.empty
    rstd_q = alloc(batch, tokens, heads, dtype=torch.float32, device=q.device)
    rstd_k = alloc(batch, tokens, heads, dtype=torch.float32, device=q.device)
    state = (torch.empty(nseq, heads, 128, 128, dtype=torch.float32, device=q.device)
             if want_state else q.new_empty((0,), dtype=torch.float32))
    ws_bytes = _fwd_workspace_bytes(1, total, heads, nseq, keep)
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    _cabi.call("kda_chunk_fwd_qknorm", 3, _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), _cabi.ptr(gate),
               _cabi.ptr(beta), _cabi.ptr(initial_state), _cabi.ptr(state) if want_state else None,
               _cabi.ptr(out), _cabi.ptr(aqk), _cabi.ptr(akk), _cabi.ptr(rstd_q), _cabi.ptr(rstd_k),
               float(eps), _cabi.ptr(cu_seqlens), _cabi.ptr(chunk_offsets), nseq, total, heads, 128, 128,
               capacity, _cabi.ptr(workspace), ws_bytes, int(keep), _cabi.stream())
    return out, state, aqk, akk, workspace, rstd_q, rstd_k


@torch.library.impl(_lib, "kda_chunk_bwd_qknorm", "CUDA")
def _chunk_bwd_qknorm(q, k, v, gate, beta, aqk, akk, saved, rstd_q, rstd_k, cu_seqlens, chunk_offsets,
                      d_output, d_final_state, initial_state, want_state_grad):
    dq, dk, dv, dg, db, dh0 = _chunk_bwd_impl(q, k, v, gate, beta, aqk, akk, cu_seqlens, chunk_offsets,
                                              d_output, d_final_state, initial_state, want_state_grad,
                                              saved=saved, rstd=(rstd_q.contiguous(), rstd_k.contiguous()))
    if dh0 is None:
        dh0 = torch.empty(0, dtype=torch.float32, device=q.device)
    return dq, dk, dv, dg, db, dh0


@torch.library.register_fake(f"{_NS}::kda_chunk_fwd_qknorm")
def _(q, k, v, gate, beta, initial_state, cu_seqlens, chunk_offsets, want_state, keep, eps):
    nseq = q.shape[0] if cu_seqlens is None else cu_seqlens.shape[0] - 1
    state = (q.new_empty((nseq, q.shape[2], q.shape[3], v.shape[-1]), dtype=torch.float32)
             if want_state else q.new_empty((0,), dtype=torch.float32))
    nbytes = _fwd_workspace_bytes(1, q.shape[0] * q.shape[1], q.shape[2], nseq, keep)
    rstd = q.new_empty(q.shape[:3], dtype=torch.float32)
    return (v.new_empty(v.shape), state, _tape(q), _tape(q), q.new_empty((nbytes,), dtype=torch.uint8),
            rstd, torch.empty_like(rstd))


@torch.library.register_fake(f"{_NS}::kda_chunk_bwd_qknorm")
def _(q, k, v, gate, beta, aqk, akk, saved, rstd_q, rstd_k, cu_seqlens, chunk_offsets, d_output,
      d_final_state, initial_state, want_state_grad):
    nseq = q.shape[0] if cu_seqlens is None else cu_seqlens.shape[0] - 1
    dh0 = (q.new_empty((nseq, q.shape[2], q.shape[3], v.shape[-1]), dtype=torch.float32)
           if want_state_grad else q.new_empty((0,), dtype=torch.float32))
    return (*_bwd_fake(q, k, v, gate, beta), dh0)


def _tape(q):
    return q.new_empty((q.shape[0], q.shape[1], q.shape[2], _CHUNK))


@torch.library.register_fake(f"{_NS}::kda_chunk_fwd")
def _(q, k, v, gate, beta, initial_state, autotune):
    return v.new_empty(v.shape), _tape(q), _tape(q)


@torch.library.register_fake(f"{_NS}::kda_chunk_fwd_with_state")
def _(q, k, v, gate, beta, initial_state, autotune):
    state = q.new_empty((q.shape[0], q.shape[2], q.shape[3], v.shape[-1]), dtype=torch.float32)
    return v.new_empty(v.shape), state, _tape(q), _tape(q)


@torch.library.register_fake(f"{_NS}::kda_chunk_fwd_ragged")
def _(q, k, v, gate, beta, initial_state, cu_seqlens, chunk_offsets, autotune):
    return v.new_empty(v.shape), _tape(q), _tape(q)


@torch.library.register_fake(f"{_NS}::kda_chunk_fwd_ragged_with_state")
def _(q, k, v, gate, beta, initial_state, cu_seqlens, chunk_offsets, autotune):
    state = q.new_empty((cu_seqlens.shape[0] - 1, q.shape[2], q.shape[3], v.shape[-1]),
                        dtype=torch.float32)
    return v.new_empty(v.shape), state, _tape(q), _tape(q)


def _bwd_fake(q, k, v, gate, beta):
    return (q.new_empty(q.shape), k.new_empty(k.shape), v.new_empty(v.shape),
            gate.new_empty(gate.shape, dtype=torch.float32),
            beta.new_empty(beta.shape, dtype=torch.float32))


@torch.library.register_fake(f"{_NS}::kda_chunk_bwd")
def _(q, k, v, gate, beta, aqk, akk, cu_seqlens, chunk_offsets, d_output, d_final_state,
      initial_state, fastmath, autotune):
    return _bwd_fake(q, k, v, gate, beta)


@torch.library.register_fake(f"{_NS}::kda_chunk_bwd_with_state_grad")
def _(q, k, v, gate, beta, aqk, akk, cu_seqlens, chunk_offsets, d_output, d_final_state,
      initial_state, fastmath, autotune):
    return (*_bwd_fake(q, k, v, gate, beta),
            torch.empty_like(initial_state, dtype=torch.float32))


@torch.library.register_fake(f"{_NS}::kda_chunk_fwd_saved")
def _(q, k, v, gate, beta, initial_state, cu_seqlens, chunk_offsets, want_state):
    nseq = q.shape[0] if cu_seqlens is None else cu_seqlens.shape[0] - 1
    state = (q.new_empty((nseq, q.shape[2], q.shape[3], v.shape[-1]), dtype=torch.float32)
             if want_state else q.new_empty((0,), dtype=torch.float32))
    nbytes = _fwd_workspace_bytes(q.shape[0], q.shape[1], q.shape[2],
                                  None if cu_seqlens is None else nseq, True)
    return (v.new_empty(v.shape), state, _tape(q), _tape(q),
            q.new_empty((nbytes,), dtype=torch.uint8))


@torch.library.register_fake(f"{_NS}::kda_chunk_bwd_saved")
def _(q, k, v, gate, beta, aqk, akk, saved, cu_seqlens, chunk_offsets, d_output, d_final_state,
      initial_state, want_state_grad):
    nseq = q.shape[0] if cu_seqlens is None else cu_seqlens.shape[0] - 1
    dh0 = (q.new_empty((nseq, q.shape[2], q.shape[3], v.shape[-1]), dtype=torch.float32)
           if want_state_grad else q.new_empty((0,), dtype=torch.float32))
    return (*_bwd_fake(q, k, v, gate, beta), dh0)


@torch.library.register_fake(f"{_NS}::kda_chunk_bwd_state_saved")
def _(gate, aqk, saved, cu_seqlens, chunk_offsets, d_output, d_final_state):
    nseq = d_output.shape[0] if cu_seqlens is None else cu_seqlens.shape[0] - 1
    return d_output.new_empty((nseq, d_output.shape[2], 128, 128), dtype=torch.float32)


# --------------------------------------------------------------------------------------------
# recurrent scan
# --------------------------------------------------------------------------------------------
def _recurrent_impl(q, k, v, gate, beta, initial_state, cu_seqlens, state_indices, want_state):
    _require_cuda(q, "the fused recurrent scan")
    batch, tokens, heads, key_dim = q.shape
    value_dim = v.shape[-1]
    nseq = batch if cu_seqlens is None else cu_seqlens.shape[0] - 1
    out = (torch.zeros if cu_seqlens is not None else torch.empty)(
        v.shape, dtype=q.dtype, device=q.device)
    final = None
    slot_stride, num_slots = heads * key_dim * value_dim, 0
    if state_indices is not None:
        slot_stride, num_slots = initial_state.stride(0), initial_state.shape[0]
    else:
        if initial_state is not None:
            initial_state = initial_state.float().contiguous()
        if want_state:
            final = torch.empty(nseq, heads, key_dim, value_dim, dtype=torch.float32,
                                device=q.device)
    _cabi.call("kda_recurrent_fwd", 1, _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), _cabi.ptr(gate),
               _cabi.ptr(beta), _cabi.dt(q), _cabi.dt(k), _cabi.dt(v), _cabi.dt(gate),
               _cabi.dt(beta), _cabi.ptr(initial_state), _cabi.ptr(final), _cabi.ptr(out),
               _cabi.dt(out), _cabi.ptr(cu_seqlens), _cabi.ptr(state_indices), slot_stride,
               num_slots, nseq, tokens, heads, key_dim, value_dim, float(key_dim) ** -0.5,
               _cabi.stream())
    return out, final


@torch.library.impl(_lib, "kda_recurrent_fwd", "CUDA")
def _recurrent_fwd(q, k, v, gate, beta, initial_state, cu_seqlens, autotune):
    return _recurrent_impl(q, k, v, gate, beta, initial_state, cu_seqlens, None, True)


@torch.library.impl(_lib, "kda_recurrent_fwd_no_state", "CUDA")
def _recurrent_fwd_no_state(q, k, v, gate, beta, initial_state, cu_seqlens, autotune):
    return _recurrent_impl(q, k, v, gate, beta, initial_state, cu_seqlens, None, False)[0]


@torch.library.impl(_lib, "kda_recurrent_fwd_paged", "CUDA")
def _recurrent_fwd_paged(q, k, v, gate, beta, state_cache, state_indices, cu_seqlens, autotune):
    return _recurrent_impl(q, k, v, gate, beta, state_cache, cu_seqlens, state_indices, False)[0]


@torch.library.register_fake(f"{_NS}::kda_recurrent_fwd")
def _(q, k, v, gate, beta, initial_state, cu_seqlens, autotune):
    nseq = q.shape[0] if cu_seqlens is None else cu_seqlens.shape[0] - 1
    state = q.new_empty(nseq, q.shape[2], q.shape[3], v.shape[-1], dtype=torch.float32)
    return torch.empty_like(v, dtype=q.dtype), state


@torch.library.register_fake(f"{_NS}::kda_recurrent_fwd_no_state")
def _(q, k, v, gate, beta, initial_state, cu_seqlens, autotune):
    return torch.empty_like(v, dtype=q.dtype)


@torch.library.register_fake(f"{_NS}::kda_recurrent_fwd_paged")
def _(q, k, v, gate, beta, state_cache, state_indices, cu_seqlens, autotune):
    return torch.empty_like(v, dtype=q.dtype)


# --------------------------------------------------------------------------------------------
# chunk offsets, gate, l2norm
# --------------------------------------------------------------------------------------------
@torch.library.impl(_lib, "kda_prepare_chunk_offsets", "CUDA")
def _prepare_chunk_offsets(cu_seqlens, tokens, chunk_size):
    out = torch.empty_like(cu_seqlens)
    _cabi.call("kda_prepare_chunk_offsets", 1, _cabi.ptr(cu_seqlens), cu_seqlens.shape[0] - 1,
               chunk_size, _cabi.ptr(out), _cabi.stream())
    return out


@torch.library.register_fake(f"{_NS}::kda_prepare_chunk_offsets")
def _(cu_seqlens, tokens, chunk_size):
    return torch.empty_like(cu_seqlens)


def _gate_chunks(raw, cu_seqlens, chunk_size):
    batch, tokens = raw.shape[0], raw.shape[1]
    if cu_seqlens is None:
        return 0, batch * ((tokens + chunk_size - 1) // chunk_size)
    nseq = cu_seqlens.shape[0] - 1
    return nseq, chunk_capacity(tokens, nseq, chunk_size)


def _gate_fwd(raw, A_log, dt_bias, cu_seqlens, chunk_offsets, chunk_size, lower_bound):
    _require_cuda(raw, "bounded_gate_cumsum")
    raw = raw.contiguous()
    batch, tokens, heads, dim = raw.shape
    nseq, chunks = _gate_chunks(raw, cu_seqlens, chunk_size)
    alloc = torch.zeros if cu_seqlens is not None else torch.empty
    out = alloc(raw.shape, dtype=torch.float32, device=raw.device)
    _cabi.call("kda_gate_cumsum_fwd", 1, _cabi.ptr(raw), _cabi.dt(raw), _cabi.ptr(A_log.contiguous()),
               _cabi.ptr(dt_bias.contiguous()), _cabi.ptr(out), _cabi.ptr(cu_seqlens),
               _cabi.ptr(chunk_offsets), nseq, batch, tokens, heads, dim, chunk_size,
               float(lower_bound), chunks, _cabi.stream())
    return out


@torch.library.impl(_lib, "kda_bounded_gate_fwd_dense", "CUDA")
def _gate_fwd_dense(raw, A_log, dt_bias, chunk_size, lower_bound):
    return _gate_fwd(raw, A_log, dt_bias, None, None, chunk_size, lower_bound)


@torch.library.impl(_lib, "kda_bounded_gate_fwd_ragged", "CUDA")
def _gate_fwd_ragged(raw, A_log, dt_bias, cu_seqlens, chunk_offsets, chunk_size, lower_bound):
    return _gate_fwd(raw, A_log, dt_bias, cu_seqlens, chunk_offsets, chunk_size, lower_bound)


@torch.library.impl(_lib, "kda_bounded_gate_bwd", "CUDA")
def _gate_bwd(raw, A_log, dt_bias, d_cumulative, cu_seqlens, chunk_offsets, chunk_size,
              lower_bound):
    raw = raw.contiguous()
    d_cumulative = d_cumulative.float().contiguous()
    batch, tokens, heads, dim = raw.shape
    nseq, chunks = _gate_chunks(raw, cu_seqlens, chunk_size)
    d_raw = (torch.zeros_like if cu_seqlens is not None else torch.empty_like)(raw)
    rows = _cabi.lib().kda_gate_bwd_partial_rows(chunks)
    pa = torch.empty(max(rows, 1), heads * dim, dtype=torch.float32, device=raw.device)
    pb = torch.empty_like(pa)
    if chunks == 0:
        pa.zero_(), pb.zero_()
    _cabi.call("kda_gate_cumsum_bwd", 1, _cabi.ptr(raw), _cabi.dt(raw), _cabi.ptr(A_log.contiguous()),
               _cabi.ptr(dt_bias.contiguous()), _cabi.ptr(d_cumulative), _cabi.ptr(d_raw),
               _cabi.ptr(pa), _cabi.ptr(pb), _cabi.ptr(cu_seqlens), _cabi.ptr(chunk_offsets), nseq,
               batch, tokens, heads, dim, chunk_size, float(lower_bound), chunks, _cabi.stream())
    dA = torch.empty(heads, dtype=torch.float32, device=raw.device)
    dbias = torch.empty(heads, dim, dtype=torch.float32, device=raw.device)
    _cabi.call("kda_gate_bwd_reduce", 1, _cabi.ptr(pa), _cabi.ptr(pb), max(rows, 1), heads, dim,
               _cabi.ptr(dA), _cabi.ptr(dbias), _cabi.stream())
    return d_raw, dA, dbias


@torch.library.register_fake(f"{_NS}::kda_bounded_gate_fwd_dense")
def _(raw, A_log, dt_bias, chunk_size, lower_bound):
    return torch.empty_like(raw, dtype=torch.float32)


@torch.library.register_fake(f"{_NS}::kda_bounded_gate_fwd_ragged")
def _(raw, A_log, dt_bias, cu_seqlens, chunk_offsets, chunk_size, lower_bound):
    return torch.empty_like(raw, dtype=torch.float32)


@torch.library.register_fake(f"{_NS}::kda_bounded_gate_bwd")
def _(raw, A_log, dt_bias, d_cumulative, cu_seqlens, chunk_offsets, chunk_size, lower_bound):
    return torch.empty_like(raw), A_log.new_empty(A_log.shape), dt_bias.new_empty(dt_bias.shape)


@torch.library.impl(_lib, "kda_l2norm_fwd", "CUDA")
def _l2norm_fwd(x, eps):
    x = x.contiguous()
    dim = x.shape[-1]
    rows = x.numel() // dim
    y = torch.empty_like(x)
    rstd = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    _cabi.call("kda_l2norm_fwd", 1, _cabi.ptr(x), _cabi.dt(x), _cabi.ptr(y), _cabi.ptr(rstd), rows,
               dim, float(eps), _cabi.stream())
    return y, rstd


@torch.library.impl(_lib, "kda_l2norm_bwd", "CUDA")
def _l2norm_bwd(y, rstd, dy):
    y, dy = y.contiguous(), dy.to(y.dtype).contiguous()
    dim = y.shape[-1]
    dx = torch.empty_like(y)
    _cabi.call("kda_l2norm_bwd", 1, _cabi.ptr(y), _cabi.ptr(rstd.contiguous()), _cabi.ptr(dy),
               _cabi.dt(y), _cabi.ptr(dx), y.numel() // dim, dim, _cabi.stream())
    return dx


@torch.library.register_fake(f"{_NS}::kda_l2norm_fwd")
def _(x, eps):
    return torch.empty_like(x), x.new_empty(x.shape[:-1], dtype=torch.float32)


@torch.library.register_fake(f"{_NS}::kda_l2norm_bwd")
def _(y, rstd, dy):
    return torch.empty_like(y)


@torch.library.impl(_lib, "kda_output_gate_fwd", "CUDA")
def _output_gate_fwd(o, gate_logits, weight, eps):
    o = o.contiguous()
    gate_logits = gate_logits.to(o.dtype).contiguous()
    dim = o.shape[-1]
    y = torch.empty_like(o)
    _cabi.call("kda_output_gate_fwd", 1, _cabi.ptr(o), _cabi.ptr(gate_logits),
               _cabi.ptr(weight.float().contiguous()), _cabi.dt(o), _cabi.ptr(y), o.numel() // dim,
               dim, float(eps), _cabi.stream())
    return y


@torch.library.impl(_lib, "kda_output_gate_bwd", "CUDA")
def _output_gate_bwd(o, gate_logits, weight, dy, eps):
    o = o.contiguous()
    gate_logits, dy = gate_logits.to(o.dtype).contiguous(), dy.to(o.dtype).contiguous()
    dim = o.shape[-1]
    rows = o.numel() // dim
    d_o, d_logits = torch.empty_like(o), torch.empty_like(o)
    partial = torch.empty(_cabi.lib().kda_output_gate_bwd_partial_rows(rows), dim,
                          dtype=torch.float32, device=o.device)
    _cabi.call("kda_output_gate_bwd", 1, _cabi.ptr(o), _cabi.ptr(gate_logits), _cabi.ptr(dy),
               _cabi.ptr(weight.float().contiguous()), _cabi.dt(o), _cabi.ptr(d_o),
               _cabi.ptr(d_logits), _cabi.ptr(partial), rows, dim, float(eps), _cabi.stream())
    return d_o, d_logits, partial.sum(0).to(weight.dtype)


@torch.library.register_fake(f"{_NS}::kda_output_gate_fwd")
def _(o, gate_logits, weight, eps):
    return torch.empty_like(o)


@torch.library.register_fake(f"{_NS}::kda_output_gate_bwd")
def _(o, gate_logits, weight, dy, eps):
    return torch.empty_like(o), torch.empty_like(o), torch.empty_like(weight)


# --------------------------------------------------------------------------------------------
# short convolution
# --------------------------------------------------------------------------------------------
_ACT = {None: 0, "silu": 1}


def _act_code(activation):
    if activation not in _ACT:
        raise ValueError(f"unknown activation {activation!r}; built in: None, 'silu'")
    return _ACT[activation]


@torch.library.impl(_lib, "short_conv_fwd", "CUDA")
def _short_conv_fwd(x, weight, cu_seqlens=None, initial_state=None, *, activation=None):
    batch, tokens, channels = x.shape
    nseq = batch if cu_seqlens is None else cu_seqlens.shape[0] - 1
    y = (torch.zeros_like if cu_seqlens is not None else torch.empty_like)(x)
    _cabi.call("kda_conv1d_fwd", 1, _cabi.ptr(x), _cabi.ptr(weight), _cabi.ptr(initial_state),
               _cabi.ptr(y), _cabi.dt(x), _cabi.ptr(cu_seqlens), nseq, batch, tokens, channels,
               weight.shape[1], _act_code(activation), _cabi.stream())
    return y


@torch.library.impl(_lib, "short_conv_bwd", "CUDA")
def _short_conv_bwd(x, weight, grad_output, cu_seqlens=None, initial_state=None, *,
                    activation=None, state_grad=False):
    batch, tokens, channels = x.shape
    width = weight.shape[1]
    nseq = batch if cu_seqlens is None else cu_seqlens.shape[0] - 1
    grad_output = grad_output.to(x.dtype).contiguous()
    dx = (torch.zeros_like if cu_seqlens is not None else torch.empty_like)(x)
    blocks = _cabi.lib().kda_conv1d_bwd_blocks(batch, tokens, int(cu_seqlens is not None))
    dw_part = torch.empty(blocks, channels, width, dtype=torch.float32, device=x.device)
    dstate = (torch.zeros(nseq, max(width - 1, 0), channels, dtype=torch.float32, device=x.device)
              if state_grad else None)
    # the width-4 kernels for 16-bit tensors need no scratch; every other case keeps dpre in fp32
    # between its two passes
    scratch = (None if width == 4 and x.element_size() == 2 else
               torch.empty(batch * tokens, channels, dtype=torch.float32, device=x.device))
    _cabi.call("kda_conv1d_bwd", 2, _cabi.ptr(x), _cabi.ptr(weight), _cabi.ptr(initial_state),
               _cabi.ptr(grad_output), _cabi.ptr(dx), _cabi.ptr(dw_part), _cabi.ptr(dstate),
               _cabi.ptr(scratch), _cabi.dt(x), _cabi.ptr(cu_seqlens), nseq, batch, tokens,
               channels, width, _act_code(activation), _cabi.stream())
    dw = torch.empty_like(weight, memory_format=torch.contiguous_format)
    _cabi.call("kda_conv1d_dw_reduce", 1, _cabi.ptr(dw_part), blocks, channels * width, _cabi.ptr(dw),
               _cabi.dt(dw), _cabi.stream())
    ds = dstate.to(x.dtype) if state_grad else x.new_empty(0)
    return dx, dw, ds


@torch.library.impl(_lib, "short_conv_decode", "CUDA")
def _short_conv_decode(x, weight, state, state_indices, *, activation=None):
    nseq, channels = x.shape
    y = torch.empty_like(x)
    _cabi.call("kda_conv1d_decode", 1, _cabi.ptr(x), _cabi.ptr(weight), _cabi.ptr(state),
               _cabi.ptr(state_indices), _cabi.ptr(y), _cabi.dt(x), nseq, state.shape[0], channels,
               weight.shape[1], _act_code(activation), _cabi.stream())
    return y


@torch.library.impl(_lib, "kda_decode_prep", "CUDA")
def _decode_prep(x, weight, conv_state, state_indices, raw_gate, A_log, dt_bias, heads, activation,
                 lower_bound, eps):
    nseq = x.shape[0]
    q = torch.empty(nseq, 1, heads, 128, dtype=x.dtype, device=x.device)
    k, v = torch.empty_like(q), torch.empty_like(q)
    gate = torch.empty(nseq, 1, heads, 128, dtype=torch.float32, device=x.device)
    raw_gate = raw_gate.contiguous()
    _cabi.call("kda_decode_prep", 1, _cabi.ptr(x), _cabi.ptr(weight), _cabi.ptr(conv_state),
               _cabi.ptr(state_indices), _cabi.ptr(raw_gate), _cabi.dt(raw_gate),
               _cabi.ptr(A_log.float().contiguous()), _cabi.ptr(dt_bias.float().contiguous()),
               _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), _cabi.ptr(gate), _cabi.dt(x), nseq, heads, 128,
               weight.shape[1], conv_state.shape[0], _act_code(activation), float(lower_bound),
               float(eps), _cabi.stream())
    return q, k, v, gate


@torch.library.register_fake(f"{_NS}::kda_decode_prep")
def _(x, weight, conv_state, state_indices, raw_gate, A_log, dt_bias, heads, activation,
      lower_bound, eps):
    q = x.new_empty((x.shape[0], 1, heads, 128))
    return q, torch.empty_like(q), torch.empty_like(q), q.new_empty(q.shape, dtype=torch.float32)


@torch.library.register_fake(f"{_NS}::short_conv_fwd")
def _(x, weight, cu_seqlens=None, initial_state=None, *, activation=None):
    return torch.empty_like(x)


@torch.library.register_fake(f"{_NS}::short_conv_bwd")
def _(x, weight, grad_output, cu_seqlens=None, initial_state=None, *, activation=None,
      state_grad=False):
    nseq = x.shape[0] if cu_seqlens is None else cu_seqlens.shape[0] - 1
    ds = (x.new_empty(nseq, weight.shape[1] - 1, x.shape[2]) if state_grad else x.new_empty(0))
    return torch.empty_like(x), torch.empty_like(weight), ds


@torch.library.register_fake(f"{_NS}::short_conv_decode")
def _(x, weight, state, state_indices, *, activation=None):
    return torch.empty_like(x)


_ops = getattr(torch.ops, _NS)
chunk_fwd_op = _ops.kda_chunk_fwd.default
chunk_fwd_with_state_op = _ops.kda_chunk_fwd_with_state.default
chunk_fwd_ragged_op = _ops.kda_chunk_fwd_ragged.default
chunk_fwd_ragged_with_state_op = _ops.kda_chunk_fwd_ragged_with_state.default
chunk_fwd_saved_op = _ops.kda_chunk_fwd_saved.default
chunk_bwd_saved_op = _ops.kda_chunk_bwd_saved.default
chunk_bwd_state_saved_op = _ops.kda_chunk_bwd_state_saved.default
chunk_fwd_qknorm_op = _ops.kda_chunk_fwd_qknorm.default
chunk_bwd_qknorm_op = _ops.kda_chunk_bwd_qknorm.default
chunk_bwd_op = _ops.kda_chunk_bwd.default
chunk_bwd_with_state_grad_op = _ops.kda_chunk_bwd_with_state_grad.default
recurrent_fwd_op = _ops.kda_recurrent_fwd.default
recurrent_fwd_no_state_op = _ops.kda_recurrent_fwd_no_state.default
recurrent_fwd_paged_op = _ops.kda_recurrent_fwd_paged.default
prepare_chunk_offsets_op = _ops.kda_prepare_chunk_offsets.default


def recurrent_forward(q, k, v, gate, beta, initial_state=None, *, cu_seqlens=None,
                      output_final_state=False, state_indices=None, autotune=True):
    """Entry of the fused scan: same checks as the reference's ``recurrent_forward``
    (attn_gym/linear/kda/ops.py:505-545)."""
    if q.shape[-1] > 256:
        raise ValueError(f"recurrent_kda requires K in [1, 256], got {q.shape[-1]}")
    if not q.is_cuda:
        raise ValueError("the fused recurrent scan requires CUDA tensors")
    tensors = (q, k, v, gate, beta) + (() if initial_state is None else (initial_state,))
    if torch.is_grad_enabled() and any(t.requires_grad for t in tensors):
        raise RuntimeError(
            "recurrent_kda is inference-only and has no backward; use chunk_kda for training "
            "or call under torch.no_grad() / torch.inference_mode()")
    q, k, v, gate, beta = (t.contiguous() for t in (q, k, v, gate, beta))
    if cu_seqlens is not None and cu_seqlens.dtype == torch.int64:
        cu_seqlens = cu_seqlens.to(torch.int32)
    if state_indices is not None:
        assert initial_state is not None
        return recurrent_fwd_paged_op(q, k, v, gate, beta, initial_state, state_indices,
                                      cu_seqlens, autotune), None
    if initial_state is not None:
        initial_state = initial_state.contiguous()
    if output_final_state:
        return recurrent_fwd_op(q, k, v, gate, beta, initial_state, cu_seqlens, autotune)
    return recurrent_fwd_no_state_op(q, k, v, gate, beta, initial_state, cu_seqlens, autotune), None
