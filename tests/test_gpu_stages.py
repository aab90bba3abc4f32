"""Stage-level parity: the intermediates of the chunked pipeline -- the tape (Aqk, A), the WY
products (w, u), the gated operands (kg, qg), the chunk-entry states h[c], v_new, and the
backward's dv2 and dh[c] -- each against the CPU oracle's value of the same quantity, with the
reference's data-derived error budget (test/test_kda_kernels.py:141-156: at most twice the error
of an independent low-precision evaluation plus two ulps of bf16 at the largest magnitude) beside
the fixed normalised tolerance.  An end-to-end check would let one stage degrade by a few times
as long as the final outputs stay inside their tolerance; this one does not.

The kernels are driven through the operator pair that keeps the intermediates
(kda_chunk_fwd_saved / kda_chunk_bwd_saved); their buffer holds, in order, w, u, kg, qg, v_new,
dv2 ([tokens, H, 128] bf16 each) and h, dh ([chunks, H, 128, 128] bf16 each)."""

import pytest
import torch

from oracle import kda_oracle as orc
from helpers import assert_budget, assert_normalised

pytestmark = pytest.mark.gpu
ops = torch.ops.kda_b200
T, H, D, C = 200, 2, 128, 64
NCH = (T + C - 1) // C


def _oracle(inp, do, dst, dtype, store_dtype=None):
    trace = {}
    res = orc.chunk_kda_grads_ref(inp["q"].float(), inp["k"].float(), inp["v"].float(), inp["cum_gate"],
                                  inp["beta"], do, inp["h0"], dst, dtype=dtype, trace=trace,
                                  store_dtype=store_dtype)
    intra = trace["intra"][0]                      # each [H, n, C, *]
    out = {name: intra[name].detach() for name in ("aqk", "akk", "w", "u", "kg", "qg")}
    out["h"] = torch.stack([h.detach() for h in trace["h"]], 1)             # [H, n, K, V]
    out["v_new"] = torch.stack([v.detach() for v in trace["v_new"]], 1)     # [H, n, C, V]
    out["dv2"] = torch.stack([v.grad for v in trace["v_new"]], 1)
    # dh[c] = gradient with respect to the state leaving chunk c
    leaving = [h.grad for h in trace["h"][1:]] + [dst[0].to(dtype)]
    out["dh"] = torch.stack(leaving, 1)
    out.update({k: res[k] for k in ("o", "state", "dq", "dk", "dv", "dg", "dbeta", "dh0")})
    return out


def _token_major(x):
    """[T, H, X] kernel layout -> [H, n, C, X] with the tail chunk zero-padded."""
    pad = NCH * C - x.shape[0]
    x = torch.nn.functional.pad(x, (0, 0, 0, 0, 0, pad))
    return x.view(NCH, C, H, x.shape[-1]).permute(2, 0, 1, 3)


def test_every_stage_against_the_oracle():
    inp = orc.make_inputs(1, T, H, D, D, seed=81, with_state=True)
    for n in ("q", "k", "v"):
        inp[n] = inp[n].bfloat16()
    gen = torch.Generator().manual_seed(82)
    do = torch.randn(1, T, H, D, generator=gen).bfloat16().float()
    dst = 0.1 * torch.randn(1, H, D, D, generator=gen)
    gold = _oracle(inp, do, dst, torch.float64)
    low = _oracle(inp, do, dst, torch.float32, store_dtype=torch.bfloat16)

    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    args = (c["q"], c["k"], c["v"], c["cum_gate"], c["beta"])
    out, state, aqk, akk, saved = ops.kda_chunk_fwd_saved(*args, c["h0"], None, None, True)
    grads = ops.kda_chunk_bwd_saved(*args, aqk, akk, saved, None, None, do.bfloat16().cuda(), dst.cuda(),
                                    c["h0"], True)
    torch.cuda.synchronize()
    nd, hs = T * H * D, NCH * H * D * D
    buf = saved[: (6 * nd + 2 * hs) * 2].view(torch.bfloat16)
    tok = {name: buf[i * nd:(i + 1) * nd].view(T, H, D)
           for i, name in enumerate(("w", "u", "kg", "qg", "v_new", "dv2"))}
    got = {name: _token_major(t.float().cpu()) for name, t in tok.items()}
    got["aqk"] = _token_major(aqk[0].float().cpu())
    got["akk"] = _token_major(akk[0].float().cpu())
    got["h"] = buf[6 * nd:6 * nd + hs].view(NCH, H, D, D).float().cpu().transpose(0, 1)
    got["dh"] = buf[6 * nd + hs:6 * nd + 2 * hs].view(NCH, H, D, D).float().cpu().transpose(0, 1)
    valid = T - (NCH - 1) * C                       # rows of the tail chunk that hold tokens
    for name in ("aqk", "akk", "w", "u", "kg", "qg", "v_new", "dv2", "h", "dh"):
        a, g, l = got[name], gold[name].float(), low[name].float()
        if name not in ("h", "dh"):                 # rows past the tail are not defined
            a, g, l = (x.clone() for x in (a, g, l))
            for x in (a, g, l):
                x[:, -1, valid:] = 0
            if name in ("aqk", "akk"):              # ... nor are the columns that pair with them
                for x in (a, g, l):
                    x[:, -1, :, valid:] = 0
        assert_normalised(a, g, 2e-2, f"stage {name}")
        assert_budget(a, g, l, f"stage {name}")
    final = {"o": out[0].float().cpu()[None], "state": state.cpu(), "dq": grads[0].float().cpu(),
             "dk": grads[1].float().cpu(), "dv": grads[2].float().cpu(), "dg": grads[3].cpu(),
             "dbeta": grads[4].cpu(), "dh0": grads[5].cpu()}
    for name, a in final.items():
        assert_normalised(a, gold[name].float(), 2e-2, f"result {name}")
        assert_budget(a, gold[name], low[name], f"result {name}")
