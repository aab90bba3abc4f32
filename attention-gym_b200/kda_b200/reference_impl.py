"""``impl="reference"``: eager fp32 PyTorch evaluation of the public KDA contract.

Plays the part of the reference's ``impl/reference.py`` + ``naive.py``: differentiable, any
device, fp32 compute with autocast disabled, packed inputs evaluated sequence by sequence after a
host read of ``cu_seqlens`` (reference: attn_gym/linear/kda/impl/reference.py:24-114,
naive.py:13-241).  It is a user-selectable implementation, never a fallback of the fused path.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def _spans(q, cu_seqlens):
    b, t = q.shape[:2]
    if cu_seqlens is None:
        return [(i, 0, t, i) for i in range(b)], b
    offs = [int(x) for x in cu_seqlens.cpu().tolist()]
    if offs[0] != 0 or any(a > c for a, c in zip(offs[:-1], offs[1:])) or offs[-1] > t:
        raise ValueError("cu_seqlens offsets must start at zero, be nondecreasing, and end within "
                         "the physical token capacity")
    return [(0, offs[i], offs[i + 1], i) for i in range(len(offs) - 1)], len(offs) - 1


def _recurrent_span(q, k, v, g, beta, state, scale):
    outs = []
    for i in range(q.shape[0]):
        state = state * torch.exp2(g[i])[..., None]
        delta = (v[i] - torch.einsum("hk,hkv->hv", k[i], state)) * beta[i][..., None]
        state = state + k[i][..., None] * delta[:, None, :]
        outs.append(torch.einsum("hk,hkv->hv", q[i] * scale, state))
    return torch.stack(outs, 0), state


def _chunk_span(q, k, v, g, beta, state, scale, chunk=64):
    t, h, kd = q.shape
    pad = (-t) % chunk
    if pad:
        q, k, v = (F.pad(x, (0, 0, 0, 0, 0, pad)) for x in (q, k, v))
        g = torch.cat((g, g[-1:].expand(pad, h, kd)), 0)
        beta = F.pad(beta, (0, 0, 0, pad))
    n = q.shape[0] // chunk
    upper = torch.triu(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device), 1)
    eye = torch.eye(chunk, dtype=q.dtype, device=q.device)
    outs = []
    for c in range(n):
        sl = slice(c * chunk, (c + 1) * chunk)
        qc, kc, vc, gc = (x[sl].transpose(0, 1) for x in (q, k, v, g))  # [H, C, D]
        bc = beta[sl].transpose(0, 1)
        rel = torch.exp2((gc[:, :, None, :] - gc[:, None, :, :]).masked_fill(upper[..., None], 0.0))
        pk = torch.einsum("hik,hjk,hijk->hij", kc * bc[..., None], kc, rel).tril(-1)
        pq = torch.einsum("hik,hjk,hijk->hij", qc * scale, kc, rel).tril()
        a = torch.linalg.solve_triangular(eye + pk, eye.expand_as(pk).clone(), upper=False)
        gam = torch.exp2(gc)
        u = a @ (vc * bc[..., None])
        w = a @ (kc * bc[..., None] * gam)
        v_new = u - w @ state
        outs.append((qc * scale * gam) @ state + pq @ v_new)
        last = gc[:, -1, :]
        state = state * torch.exp2(last)[..., None] + (
            kc * torch.exp2(last[:, None, :] - gc)).transpose(-1, -2) @ v_new
    return torch.cat(outs, 1).transpose(0, 1)[:t], state


def reference_kda(kind, q, k, v, gate, beta, initial_state, cu_seqlens, output_final_state):
    out_dtype = q.dtype
    qf, kf, vf, gf, bf = (x.float() for x in (q, k, v, gate, beta))
    h0 = None if initial_state is None else initial_state.float()
    b, t, h, kd = q.shape
    vd = v.shape[-1]
    scale = kd ** -0.5
    span_fn = _recurrent_span if kind == "recurrent" else _chunk_span
    with torch.autocast(device_type=q.device.type, enabled=False):
        spans, nseq = _spans(q, cu_seqlens)
        rows = [[] for _ in range(b)]
        cursor = [0] * b
        finals = []
        for row, bos, eos, seq in spans:
            s0 = (qf.new_zeros(h, kd, vd) if h0 is None else h0[seq])
            if eos == bos:
                finals.append(s0)
                continue
            o, s1 = span_fn(qf[row, bos:eos], kf[row, bos:eos], vf[row, bos:eos], gf[row, bos:eos],
                            bf[row, bos:eos], s0, scale)
            rows[row].append(o)
            cursor[row] = eos
            finals.append(s1)
        outs = []
        for row in range(b):
            if cursor[row] < t:
                rows[row].append(qf.new_zeros(t - cursor[row], h, vd))
            outs.append(torch.cat(rows[row], 0))
    out = torch.stack(outs, 0).to(out_dtype)
    return out, (torch.stack(finals, 0) if output_final_state else None)


__all__ = ["reference_kda"]
