"""CPU oracle for the KDA (Kimi Delta Attention) gated delta-rule path.

TEST INFRASTRUCTURE ONLY.  Nothing under ``oracle/`` is part of the product: the
shipped library never imports it.  Only the test-suite, the smoke check and the
CPU-baseline leg of the benchmark may call it, and only as the checker or as the
timed CPU port -- never as the thing that is shipped.

Every function is an independent restatement (eager PyTorch on CPU, fp32 or fp64)
of the mathematics of the reference implementation in meta-pytorch/attention-gym;
each docstring names the reference file:line it follows.  The restatement is
pinned against the reference itself: ``tests/golden/make_golden.py`` imports the
reference's own ``attn_gym.linear.kda`` oracles on CPU, runs them on seeded inputs
and stores input seeds plus outputs under ``tests/golden/``;
``tests/test_oracle_golden.py`` checks every function here against those vectors.

Conventions (identical to the reference):
  * gates are log2 decays: ``a_t = 2 ** g_t``;
  * ``chunk_kda`` consumes the inclusive *chunk-local cumulative* log2 gate,
    ``recurrent_kda`` the per-token log2 gate;
  * per token:  S <- diag(2^g) S ; d = beta (v - S^T k) ; S <- S + k d^T ; o = scale S^T q;
  * state layout ``[N, H, K, V]``; ``scale = K ** -0.5``.
"""

from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

LOG2E = 1.4426950408889634
LN2 = 0.6931471805599453
CHUNK = 64


def _compute_dtype(*tensors: torch.Tensor) -> torch.dtype:
    dtype = torch.float32
    for t in tensors:
        if t is not None:
            dtype = torch.promote_types(dtype, t.dtype)
    return dtype


def _offsets(cu_seqlens, tokens: int) -> list:
    if cu_seqlens is None:
        return [0, tokens]
    return [int(x) for x in cu_seqlens.tolist()]


# --------------------------------------------------------------------------------------
# token recurrence  (reference: attn_gym/linear/kda/naive.py:13-96)
# --------------------------------------------------------------------------------------
def recurrent_kda_ref(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    gate: torch.Tensor,
    beta: torch.Tensor,
    initial_state: Optional[torch.Tensor] = None,
    cu_seqlens: Optional[torch.Tensor] = None,
    scale: Optional[float] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """O(T) delta-rule recurrence; returns (output in q.dtype, final state in compute dtype).

    Follows naive.py:84-96 (dense) and naive.py:45-75 (packed: the recurrence restarts
    at each boundary, empty sequences pass their state through, rows past the terminal
    offset stay zero).  ``gate`` is the per-token log2 decay.
    """
    b, t, h, kd = q.shape
    vd = v.shape[-1]
    dt = _compute_dtype(q, k, v, gate, beta, initial_state)
    sc = kd ** -0.5 if scale is None else scale
    if cu_seqlens is None:
        spans = [(i, 0, t, i) for i in range(b)]
        nseq = b
    else:
        offs = _offsets(cu_seqlens, t)
        spans = [(0, offs[i], offs[i + 1], i) for i in range(len(offs) - 1)]
        nseq = len(offs) - 1
    out = torch.zeros(b, t, h, vd, dtype=dt)
    state = (
        torch.zeros(nseq, h, kd, vd, dtype=dt)
        if initial_state is None
        else initial_state.to(dt).clone()
    )
    qf, kf, vf, gf, bf = (x.to(dt) for x in (q, k, v, gate, beta))
    finals = []
    for row, bos, eos, seq in spans:
        s = state[seq]
        for i in range(bos, eos):
            s = s * torch.exp2(gf[row, i])[..., None]
            delta = (vf[row, i] - torch.einsum("hk,hkv->hv", kf[row, i], s)) * bf[row, i][..., None]
            s = s + kf[row, i][..., None] * delta[:, None, :]
            out[row, i] = torch.einsum("hk,hkv->hv", qf[row, i] * sc, s)
        finals.append(s)
    return out.to(q.dtype), torch.stack(finals, 0)


# --------------------------------------------------------------------------------------
# chunked form  (reference: attn_gym/linear/kda/naive.py:99-241)
# --------------------------------------------------------------------------------------
def _round_through(x, dtype):
    """Round ``x`` to ``dtype`` and back; the gradient passes straight through the rounding."""
    if dtype is None:
        return x
    return x + (x.detach().to(dtype).to(x.dtype) - x.detach())


def _chunk_intra(qc, kc, vc, gc, bc, sc, store_dtype=None):
    """Intra-chunk quantities for a batch of chunks ``[..., C, D]`` (naive.py:111-131).

    Returns (Aqk, A, w, u, kg, qg, d_last) with
      P_ij = sum_c k_ic k_jc 2^{G_ic - G_jc};  L = stril(beta_i P_ij);  A = (I + L)^-1
      Aqk = scale * tril(q-k pairwise product);  w = A (beta k 2^G);  u = A (beta v)
      kg = k 2^{G_last - G};  qg = scale q 2^G.
    """
    c = qc.shape[-2]
    rel = gc[..., :, None, :] - gc[..., None, :, :]
    upper = torch.triu(torch.ones(c, c, dtype=torch.bool), 1)
    rel = torch.exp2(rel.masked_fill(upper[..., None], 0.0))
    pk = torch.einsum("...ik,...jk,...ijk->...ij", kc, kc, rel)
    pq = torch.einsum("...ik,...jk,...ijk->...ij", qc, kc, rel)
    eye = torch.eye(c, dtype=qc.dtype)
    lower = (pk * bc[..., None]).tril(-1)
    a = torch.linalg.solve_triangular(eye + lower, eye.expand_as(lower).clone(), upper=False)
    aqk = (pq * sc).tril()
    gam = torch.exp2(gc)
    a = _round_through(a, store_dtype)
    w = a @ _round_through(kc * bc[..., None] * gam, store_dtype)
    u = a @ _round_through(vc * bc[..., None], store_dtype)
    d_last = gc[..., -1, :]
    kg = kc * torch.exp2(d_last[..., None, :] - gc)
    qg = qc * gam * sc
    return aqk, a, w, u, kg, qg, d_last


def _chunk_sequence(q, k, v, g, beta, state, sc, chunk, trace=None, store_dtype=None):
    """One sequence ``[T, H, D]`` -> (o [T,H,V], final state [H,K,V]).

    Pads the tail chunk the way naive.py:196-201 does (zero q/k/v/beta, the last
    cumulative gate row repeated) so the padded rows neither write nor decay.

    ``store_dtype`` (e.g. bfloat16) turns this into the *low-precision reference* of the
    reference's stage tests (test/test_kda_kernels.py:722-756 ``_fwd_h_ref``, :141-156): the
    intermediates a kernel pipeline stores in 16 bits -- Aqk, A, w, u, kg, qg, v_new and the
    state as a matrix-product operand -- are rounded to that type, the fp32 state itself is not.
    """
    t, h, kd = q.shape
    vd = v.shape[-1]
    pad = (-t) % chunk
    if pad:
        q, k, v = (F.pad(x, (0, 0, 0, 0, 0, pad)) for x in (q, k, v))
        g = torch.cat((g, g[-1:].expand(pad, h, kd)), 0)
        beta = F.pad(beta, (0, 0, 0, pad))
    n = q.shape[0] // chunk

    def split(x):  # [T,H,D] -> [H, n, C, D]
        return x.reshape(n, chunk, h, x.shape[-1]).permute(2, 0, 1, 3)

    qc, kc, vc, gc = map(split, (q, k, v, g))
    bc = beta.reshape(n, chunk, h).permute(2, 0, 1)
    outs = []
    group = max(1, 64 // max(1, h))  # bound the [.., C, C, K] pairwise tensor (~130 MB)
    intra = []
    for c0 in range(0, n, group):
        sl = slice(c0, min(n, c0 + group))
        intra.append(_chunk_intra(qc[:, sl], kc[:, sl], vc[:, sl], gc[:, sl], bc[:, sl], sc,
                                  store_dtype))
    aqk, a, w, u, kg, qg, d_last = (torch.cat([x[i] for x in intra], 1) for i in range(7))
    if store_dtype is not None:
        aqk, w, u, kg, qg = (_round_through(x, store_dtype) for x in (aqk, w, u, kg, qg))
    if trace is not None:
        trace.setdefault("intra", []).append(
            {"aqk": aqk, "akk": a, "w": w, "u": u, "kg": kg, "qg": qg})
    for c in range(n):
        operand = _round_through(state, store_dtype)
        v_new = _round_through(u[:, c] - w[:, c] @ operand, store_dtype)
        if trace is not None:
            if state.requires_grad:
                state.retain_grad()
                v_new.retain_grad()
            trace.setdefault("h", []).append(state)
            trace.setdefault("v_new", []).append(v_new)
        outs.append(qg[:, c] @ operand + aqk[:, c] @ v_new)
        state = state * torch.exp2(d_last[:, c])[..., None] + kg[:, c].transpose(-1, -2) @ v_new
    o = torch.stack(outs, 1).reshape(h, n * chunk, vd).permute(1, 0, 2)[:t]
    return o, state


def chunk_kda_ref(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cumulative_gate: torch.Tensor,
    beta: torch.Tensor,
    initial_state: Optional[torch.Tensor] = None,
    cu_seqlens: Optional[torch.Tensor] = None,
    scale: Optional[float] = None,
    chunk_size: int = CHUNK,
    trace: Optional[dict] = None,
    store_dtype: Optional[torch.dtype] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Chunk-parallel KDA from the chunk-local cumulative log2 gate; differentiable.

    Follows naive.py:141-241 for the dense form and kda/impl/reference.py:24-76 for the
    packed form (sequence-relative chunks, empty sequences pass state through, rows
    past the terminal offset are zero).  Returns (output in q.dtype, final state).
    """
    b, t, h, kd = q.shape
    vd = v.shape[-1]
    dt = _compute_dtype(q, k, v, cumulative_gate, beta, initial_state)
    sc = kd ** -0.5 if scale is None else scale
    qf, kf, vf, gf, bf = (x.to(dt) for x in (q, k, v, cumulative_gate, beta))
    if cu_seqlens is None:
        spans = [(i, 0, t, i) for i in range(b)]
        nseq = b
    else:
        offs = _offsets(cu_seqlens, t)
        spans = [(0, offs[i], offs[i + 1], i) for i in range(len(offs) - 1)]
        nseq = len(offs) - 1
    rows = [[] for _ in range(b)]
    cursor = [0] * b
    finals = []
    for row, bos, eos, seq in spans:
        s0 = (
            torch.zeros(h, kd, vd, dtype=dt)
            if initial_state is None
            else initial_state[seq].to(dt)
        )
        if eos == bos:
            finals.append(s0)
            continue
        o, s1 = _chunk_sequence(
            qf[row, bos:eos], kf[row, bos:eos], vf[row, bos:eos], gf[row, bos:eos],
            bf[row, bos:eos], s0, sc, chunk_size, trace, store_dtype,
        )
        rows[row].append(o)
        cursor[row] = eos
        finals.append(s1)
    outs = []
    for row in range(b):
        if cursor[row] < t:
            rows[row].append(torch.zeros(t - cursor[row], h, vd, dtype=dt))
        outs.append(torch.cat(rows[row], 0))
    return torch.stack(outs, 0).to(q.dtype), torch.stack(finals, 0)


def chunk_kda_grads_ref(q, k, v, cumulative_gate, beta, d_output, initial_state=None,
                        d_final_state=None, cu_seqlens=None, dtype=torch.float64, trace=None,
                        store_dtype=None):
    """Gradients of :func:`chunk_kda_ref` by autograd in ``dtype``.

    Returns dict(o, state, dq, dk, dv, dg, dbeta, dh0).  ``dg`` is the gradient with
    respect to the *cumulative* gate, as the reference op returns it
    (kda/ops.py:44-58; bwd/cute/chunk_kda_bwd.py:129-143).
    """
    leaves = [x.detach().to(dtype).requires_grad_(True) for x in (q, k, v, cumulative_gate, beta)]
    h0 = None if initial_state is None else initial_state.detach().to(dtype).requires_grad_(True)
    o, st = chunk_kda_ref(*leaves, initial_state=h0, cu_seqlens=cu_seqlens, trace=trace,
                          store_dtype=store_dtype)
    loss = (o * d_output.to(dtype)).sum()
    if d_final_state is not None:
        loss = loss + (st * d_final_state.to(dtype)).sum()
    wrt = leaves + ([h0] if h0 is not None else [])
    grads = torch.autograd.grad(loss, wrt, allow_unused=True)
    names = ["dq", "dk", "dv", "dg", "dbeta"] + (["dh0"] if h0 is not None else [])
    res = {"o": o.detach(), "state": st.detach()}
    for n, gr, leaf in zip(names, grads, wrt):
        res[n] = torch.zeros_like(leaf) if gr is None else gr
    return res


# --------------------------------------------------------------------------------------
# pre-ops
# --------------------------------------------------------------------------------------
def chunk_local_cumsum_ref(x, chunk_size, reverse=False, cu_seqlens=None):
    """Cumulative sum over time (dim 1) restarting at every chunk and sequence boundary.

    Follows naive.py:311-342.  Rows past the terminal offset are returned as zero.
    """
    b, t = x.shape[:2]
    out = torch.zeros_like(x)
    offs = _offsets(cu_seqlens, t)
    for bos, eos in zip(offs[:-1], offs[1:]):
        for c0 in range(bos, eos, chunk_size):
            c1 = min(eos, c0 + chunk_size)
            seg = x[:, c0:c1]
            out[:, c0:c1] = seg.flip(1).cumsum(1).flip(1) if reverse else seg.cumsum(1)
    return out


def bounded_gate_cumsum_ref(raw_gate, A_log, dt_bias, chunk_size=CHUNK, lower_bound=-5.0,
                            cu_seqlens=None):
    """``G = log2(e) * chunk_cumsum(lower_bound * sigmoid(exp(A_log) * (raw + dt_bias)))``.

    Follows naive.py:345-385 with the fused path's fixed log2(e) post-scale
    (fwd/triton/gate_fwd.py:59-132).  fp32 (fp64 for fp64 input) math; fp32 result.
    """
    dt = _compute_dtype(raw_gate)
    z = raw_gate.to(dt) + dt_bias.to(dt)
    gate = lower_bound * torch.sigmoid(A_log.to(dt).exp().view(1, 1, -1, 1) * z)
    return chunk_local_cumsum_ref(gate, chunk_size, False, cu_seqlens) * LOG2E


def bounded_gate_cumsum_bwd_ref(raw_gate, A_log, dt_bias, d_cumulative, chunk_size=CHUNK,
                                lower_bound=-5.0, cu_seqlens=None):
    """(d_raw, dA_log, d_dt_bias) of :func:`bounded_gate_cumsum_ref` (naive.py:388-455).

    The adjoint of the forward prefix sum is a reverse prefix sum, then the pointwise
    derivative ``lb * a * s (1 - s)`` with ``s = sigmoid(a z)``; ``dA_log = sum d_raw z``
    per head, ``d_dt_bias = sum over tokens of d_raw`` (bwd/triton/gate_bwd.py:9-15).
    """
    dt = _compute_dtype(raw_gate, d_cumulative)
    dgate = chunk_local_cumsum_ref(d_cumulative.to(dt), chunk_size, True, cu_seqlens) * LOG2E
    a = A_log.to(dt).exp().view(1, 1, -1, 1)
    z = raw_gate.to(dt) + dt_bias.to(dt)
    s = torch.sigmoid(a * z)
    d_raw = dgate * lower_bound * a * s * (1 - s)
    if cu_seqlens is not None:
        end = _offsets(cu_seqlens, raw_gate.shape[1])[-1]
        d_raw[:, end:] = 0
    dA_log = (d_raw * z).sum((0, 1, 3))
    d_bias = d_raw.sum((0, 1))
    return d_raw, dA_log, d_bias


def l2norm_ref(x, eps=1e-6):
    """``y = x * rsqrt(sum(x^2) + eps)`` over the last dim (naive.py:276-291)."""
    dt = _compute_dtype(x)
    xc = x.to(dt)
    rstd = torch.rsqrt((xc * xc).sum(-1, keepdim=True) + eps)
    return (xc * rstd).to(x.dtype), rstd


def l2norm_bwd_ref(y, rstd, dy):
    """``dx = rstd * (dy - y <dy, y>)`` (naive.py:294-308)."""
    dt = _compute_dtype(y)
    yc, dyc = y.to(dt), dy.to(dt)
    return (rstd.to(dt) * (dyc - yc * (dyc * yc).sum(-1, keepdim=True))).to(y.dtype)


def gated_output_norm_ref(o, gate_logits, weight, eps=1e-5):
    """``o * rsqrt(mean(o^2) + eps) * weight * sigmoid(gate_logits)`` over the last dim: the
    layer's output epilogue (examples/kda_training.py:507-517 RMSNorm, :519-539 sigmoid gate and
    product), in fp32 (fp64 for fp64 input) without intermediate rounding."""
    dt = _compute_dtype(o)
    oc = o.to(dt)
    rstd = torch.rsqrt((oc * oc).mean(-1, keepdim=True) + eps)
    return (oc * rstd * weight.to(dt) * torch.sigmoid(gate_logits.to(dt))).to(o.dtype)


def causal_conv1d_ref(x, weight, activation=None, cu_seqlens=None, initial_state=None):
    """Depthwise causal convolution ``y[t,c] = act(sum_j w[c,j] x[t-(W-1)+j, c])``.

    ``x [B,T,C]``, ``weight [C,W]``, history ``initial_state [N,W-1,C]`` (oldest first)
    feeding negative positions (kda/short_conv/cute.py:3464-3520).  Returns
    (y in x.dtype, final history [N,W-1,C]); packed rows past the terminal offset are zero.
    """
    b, t, c = x.shape
    wd = weight.shape[1]
    dt = _compute_dtype(x)
    xf, wf = x.to(dt), weight.to(dt)
    offs = _offsets(cu_seqlens, t)
    spans = (
        [(i, 0, t, i) for i in range(b)]
        if cu_seqlens is None
        else [(0, offs[i], offs[i + 1], i) for i in range(len(offs) - 1)]
    )
    y = torch.zeros(b, t, c, dtype=dt)
    finals = []
    for row, bos, eos, seq in spans:
        hist = (
            torch.zeros(wd - 1, c, dtype=dt)
            if initial_state is None
            else initial_state[seq].to(dt)
        )
        ext = torch.cat((hist, xf[row, bos:eos]), 0)
        n = eos - bos
        acc = torch.zeros(n, c, dtype=dt)
        for j in range(wd):
            acc = acc + ext[j:j + n] * wf[:, j]
        y[row, bos:eos] = acc
        finals.append(ext[ext.shape[0] - (wd - 1):])
    if activation == "silu":
        y = F.silu(y)
        if cu_seqlens is not None:
            y[:, offs[-1]:] = 0
    elif activation is not None:
        raise ValueError(f"unknown activation {activation!r}")
    return y.to(x.dtype), torch.stack(finals, 0).to(x.dtype)


# --------------------------------------------------------------------------------------
# context-parallel composition: h_out = M h_in + b  per slice
# --------------------------------------------------------------------------------------
def slice_transition_ref(k, cumulative_gate_or_gate, beta, per_token_gate: bool = True):
    """Dense per-head transition ``M = prod_t (I - beta_t k_t k_t^T) diag(2^{g_t})`` of a slice.

    ``k, gate [T,H,K]``, ``beta [T,H]`` with per-token log2 gates.  Returns ``[H,K,K]`` so
    that the state leaving the slice is ``M @ h_in + b`` with ``b`` the zero-input state.
    The reference has no context parallelism (docs/linear.md:220-222); this restates the
    recurrence of naive.py:84-96 applied to an identity initial state with ``v = 0``.
    """
    t, h, kd = k.shape
    dt = _compute_dtype(k, cumulative_gate_or_gate, beta)
    m = torch.eye(kd, dtype=dt).expand(h, kd, kd).clone()
    kf, gf, bf = k.to(dt), cumulative_gate_or_gate.to(dt), beta.to(dt)
    for i in range(t):
        m = m * torch.exp2(gf[i])[..., None]
        m = m - bf[i][:, None, None] * kf[i][..., None] * torch.einsum("hk,hkj->hj", kf[i], m)[:, None, :]
    return m


# --------------------------------------------------------------------------------------
# seeded synthetic inputs with the benchmark configurations' shapes and distributions
# --------------------------------------------------------------------------------------
def make_inputs(batch, tokens, heads, key_dim, value_dim, seed=0, dtype=torch.float32,
                with_state=False, lengths: Optional[Sequence[int]] = None):
    """q,k ~ N(0,1) L2-normalised; v ~ N(0,1); g = logsigmoid(N(0,1)) (nats);
    beta = sigmoid(N(0,1)); optional h0 ~ N(0, 0.02).  One generator per tensor.

    Returns a dict with q,k,v (``dtype``), ``gate_nat`` (fp32 per-token natural-log gate),
    ``gate_log2`` (per token, log2), ``cum_gate`` (chunk-local cumulative log2, restarting at
    sequence starts), ``beta`` (fp32), ``h0``, ``cu_seqlens`` (int32 or None).
    """
    def gen(i):
        return torch.Generator().manual_seed(seed * 1000 + i)

    q = torch.randn(batch, tokens, heads, key_dim, generator=gen(1))
    k = torch.randn(batch, tokens, heads, key_dim, generator=gen(2))
    v = torch.randn(batch, tokens, heads, value_dim, generator=gen(3))
    q = q / q.norm(dim=-1, keepdim=True)
    k = k / k.norm(dim=-1, keepdim=True)
    g_nat = F.logsigmoid(torch.randn(batch, tokens, heads, key_dim, generator=gen(4)))
    beta = torch.sigmoid(torch.randn(batch, tokens, heads, generator=gen(5)))
    cu = None
    nseq = batch
    if lengths is not None:
        assert batch == 1 and sum(lengths) <= tokens
        offs = [0]
        for n in lengths:
            offs.append(offs[-1] + int(n))
        cu = torch.tensor(offs, dtype=torch.int32)
        nseq = len(lengths)
    h0 = None
    if with_state:
        h0 = 0.02 * torch.randn(nseq, heads, key_dim, value_dim, generator=gen(6))
    g2 = g_nat * LOG2E
    cum = chunk_local_cumsum_ref(g2, CHUNK, False, cu)
    return {
        "q": q.to(dtype), "k": k.to(dtype), "v": v.to(dtype), "gate_nat": g_nat,
        "gate_log2": g2, "cum_gate": cum, "beta": beta, "h0": h0, "cu_seqlens": cu,
    }


def draw_lengths(num_sequences, low, high, seed=0):
    """Sequence lengths uniform-int in [low, high] from the seed."""
    gen = torch.Generator().manual_seed(seed * 1000 + 77)
    return torch.randint(low, high + 1, (num_sequences,), generator=gen).tolist()


__all__ = [
    "recurrent_kda_ref", "chunk_kda_ref", "chunk_kda_grads_ref", "chunk_local_cumsum_ref",
    "bounded_gate_cumsum_ref", "bounded_gate_cumsum_bwd_ref", "l2norm_ref", "l2norm_bwd_ref",
    "causal_conv1d_ref", "slice_transition_ref", "make_inputs", "draw_lengths",
    "LOG2E", "LN2", "CHUNK",
]
