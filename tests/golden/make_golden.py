"""Generate the golden fixtures in this folder from the reference implementation.

Run where the reference checkout is available (it is imported, never copied):

    PYTHONPATH=<reference checkout> python tests/golden/make_golden.py

It imports the reference's own CPU oracles (``attn_gym.linear.kda.naive`` and the public
``chunk_kda`` / ``recurrent_kda`` with ``impl="reference"``), runs them on seeded inputs,
and writes inputs + outputs as ``.npz`` files.  The tests only read the ``.npz`` files, so
they run on machines that do not have the reference.
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle.kda_oracle import LOG2E, make_inputs  # noqa: E402  (input factory only)


def _np(d):
    return {k: (v.detach().numpy() if torch.is_tensor(v) else np.asarray(v)) for k, v in d.items()
            if v is not None}


def _save(name, **arrays):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **_np(arrays))
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")


def main():
    from attn_gym.linear.kda import chunk_kda, recurrent_kda
    from attn_gym.linear.kda import naive

    torch.set_num_threads(8)

    # 1. recurrent, dense, with an initial state ------------------------------------------
    inp = make_inputs(2, 40, 2, 16, 24, seed=11, with_state=True)
    o, st = recurrent_kda(inp["q"], inp["k"], inp["v"], inp["gate_log2"], inp["beta"], inp["h0"],
                          output_final_state=True, impl="reference")
    _save("recurrent_dense", q=inp["q"], k=inp["k"], v=inp["v"], gate=inp["gate_log2"],
          beta=inp["beta"], h0=inp["h0"], o=o, state=st)

    # 2. recurrent, packed with an empty sequence and an inactive suffix --------------------
    inp = make_inputs(1, 40, 2, 16, 24, seed=12, with_state=True, lengths=[5, 0, 17, 9])
    o, st = recurrent_kda(inp["q"], inp["k"], inp["v"], inp["gate_log2"], inp["beta"], inp["h0"],
                          cu_seqlens=inp["cu_seqlens"], output_final_state=True, impl="reference")
    _save("recurrent_packed", q=inp["q"], k=inp["k"], v=inp["v"], gate=inp["gate_log2"],
          beta=inp["beta"], h0=inp["h0"], cu_seqlens=inp["cu_seqlens"], o=o, state=st)

    # 3. chunked, dense with a partial tail chunk, forward + all gradients ------------------
    inp = make_inputs(2, 130, 2, 32, 32, seed=13, with_state=True)
    leaves = [inp[n].clone().requires_grad_(True) for n in ("q", "k", "v", "cum_gate", "beta")]
    h0 = inp["h0"].clone().requires_grad_(True)
    o, st = chunk_kda(*leaves, h0, output_final_state=True, impl="reference")
    gen = torch.Generator().manual_seed(99)
    do = torch.randn(o.shape, generator=gen)
    dst = 0.1 * torch.randn(st.shape, generator=gen)
    grads = torch.autograd.grad((o * do).sum() + (st * dst).sum(), leaves + [h0])
    _save("chunk_dense", q=inp["q"], k=inp["k"], v=inp["v"], cum_gate=inp["cum_gate"],
          beta=inp["beta"], h0=inp["h0"], o=o, state=st, do=do, dstate=dst,
          dq=grads[0], dk=grads[1], dv=grads[2], dg=grads[3], dbeta=grads[4], dh0=grads[5])

    # 4. chunked, packed: lengths straddling chunk boundaries, an empty sequence, a suffix ---
    inp = make_inputs(1, 200, 2, 32, 32, seed=14, with_state=True, lengths=[65, 63, 0, 30])
    leaves = [inp[n].clone().requires_grad_(True) for n in ("q", "k", "v", "cum_gate", "beta")]
    h0 = inp["h0"].clone().requires_grad_(True)
    o, st = chunk_kda(*leaves, h0, cu_seqlens=inp["cu_seqlens"], output_final_state=True,
                      impl="reference")
    do = torch.randn(o.shape, generator=gen)
    dst = 0.1 * torch.randn(st.shape, generator=gen)
    grads = torch.autograd.grad((o * do).sum() + (st * dst).sum(), leaves + [h0])
    _save("chunk_packed", q=inp["q"], k=inp["k"], v=inp["v"], cum_gate=inp["cum_gate"],
          beta=inp["beta"], h0=inp["h0"], cu_seqlens=inp["cu_seqlens"], o=o, state=st, do=do,
          dstate=dst, dq=grads[0], dk=grads[1], dv=grads[2], dg=grads[3], dbeta=grads[4],
          dh0=grads[5])

    # 5. benchmark configuration 0 (B1 H4 T512 K=V=64 fp32): outputs only, inputs by seed ----
    inp = make_inputs(1, 512, 4, 64, 64, seed=0)
    o_r, st_r = recurrent_kda(inp["q"], inp["k"], inp["v"], inp["gate_log2"], inp["beta"],
                              output_final_state=True, impl="reference")
    o_c, st_c = chunk_kda(inp["q"], inp["k"], inp["v"], inp["cum_gate"], inp["beta"],
                          output_final_state=True, impl="reference")
    # the natural-log statement of the benchmark configuration, S_t=(I-b k k^T)Diag(exp g)S+b k v^T
    s = torch.zeros(4, 64, 64, dtype=torch.float64)
    o_nat = torch.zeros(512, 4, 64, dtype=torch.float64)
    qd, kd, vd = (inp[n][0].double() for n in ("q", "k", "v"))
    gd, bd = inp["gate_nat"][0].double(), inp["beta"][0].double()
    for t in range(512):
        s = s * gd[t].exp()[..., None]
        s = s + bd[t][:, None, None] * kd[t][..., None] * (
            vd[t] - torch.einsum("hk,hkv->hv", kd[t], s))[:, None, :]
        o_nat[t] = torch.einsum("hk,hkv->hv", qd[t] * 64 ** -0.5, s)
    sums = {n: np.array([float(inp[n].double().sum()), float(inp[n].double().abs().sum())])
            for n in ("q", "k", "v", "gate_log2", "beta")}
    # full recurrent output; the other two formulations every 8th token (they agree to 1e-6)
    _save("config0", o_recurrent=o_r, state_recurrent=st_r, o_chunk_s8=o_c[:, ::8],
          state_chunk=st_c, o_natural_fp64_s8=o_nat.float()[::8], state_natural_fp64=s.float(),
          **{"sum_" + n: val for n, val in sums.items()})

    # 6. gate pre-op: forward and backward references ---------------------------------------
    gen = torch.Generator().manual_seed(21)
    raw = torch.randn(2, 150, 3, 32, generator=gen).bfloat16()
    A_log = 0.3 * torch.randn(3, generator=gen)
    dt_bias = 0.5 * torch.randn(3, 32, generator=gen)
    dcum = torch.randn(2, 150, 3, 32, generator=gen)
    fwd = naive.gate_fwd_ref(raw, A_log, dt_bias, -5.0, LOG2E, False, 64, None)
    draw, dA, dbias = naive.fused_gate_bwd_ref(raw, A_log, dt_bias, dcum, -5.0, LOG2E, 64)
    cu = torch.tensor([0, 70, 70, 131], dtype=torch.int32)
    fwd_p = naive.gate_fwd_ref(raw[:1, :131], A_log, dt_bias, -5.0, LOG2E, False, 64, cu)
    cs = naive.chunk_cumsum_ref(dcum, 16, reverse=True)
    _save("gate", raw=raw.float(), A_log=A_log, dt_bias=dt_bias, dcum=dcum, fwd=fwd,
          d_raw=draw, dA_log=dA, d_dt_bias=dbias, cu_seqlens=cu, fwd_packed=fwd_p,
          revcumsum16=cs)

    # 7. l2norm forward / backward ------------------------------------------------------------
    x = torch.randn(3, 7, 2, 48, generator=gen)
    dy = torch.randn(3, 7, 2, 48, generator=gen)
    y = naive.l2norm_fwd_ref(x)
    rstd = torch.rsqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    dx = naive.l2norm_bwd_ref(y, rstd, dy)
    _save("l2norm", x=x, dy=dy, y=y, rstd=rstd, dx=dx)

    # 8. short convolution: the reference tests' own oracle is F.conv1d (+ SiLU) --------------
    #    (test/test_kda_short_conv_cute.py:49-55)
    x = torch.randn(2, 37, 24, generator=gen).requires_grad_(True)
    w = torch.randn(24, 4, generator=gen).requires_grad_(True)
    hist = torch.randn(2, 3, 24, generator=gen).requires_grad_(True)
    ext = torch.cat((hist, x), 1)
    y = F.silu(F.conv1d(ext.transpose(1, 2), w[:, None], groups=24).transpose(1, 2))
    dy = torch.randn(y.shape, generator=gen)
    dx, dw, dhist = torch.autograd.grad((y * dy).sum(), (x, w, hist))
    _save("conv", x=x, w=w, hist=hist, y=y, dy=dy, dx=dx, dw=dw, dhist=dhist,
          final=ext[:, -3:])


if __name__ == "__main__":
    main()
