"""Pin the CPU oracle against vectors produced by the reference's own CPU implementation.

The fixtures in tests/golden/*.npz were written by tests/golden/make_golden.py, which imports
the reference (attn_gym.linear.kda, impl="reference", and its naive.* helpers).
"""

import torch

from oracle import kda_oracle as orc


def _close(a, b, atol, rtol=1e-4):
    torch.testing.assert_close(a.float(), b.float(), atol=atol, rtol=rtol)


def test_recurrent_dense(golden):
    g = golden("recurrent_dense")
    o, st = orc.recurrent_kda_ref(g["q"], g["k"], g["v"], g["gate"], g["beta"], g["h0"])
    _close(o, g["o"], 1e-6)
    _close(st, g["state"], 1e-6)


def test_recurrent_packed(golden):
    g = golden("recurrent_packed")
    o, st = orc.recurrent_kda_ref(g["q"], g["k"], g["v"], g["gate"], g["beta"], g["h0"],
                                  cu_seqlens=g["cu_seqlens"])
    _close(o, g["o"], 1e-6)
    _close(st, g["state"], 1e-6)
    assert torch.equal(st[1], g["h0"][1])  # the empty sequence passes its state through
    assert o[:, 31:].abs().max() == 0  # rows past the terminal offset stay zero


def test_chunk_dense_forward_and_grads(golden):
    g = golden("chunk_dense")
    res = orc.chunk_kda_grads_ref(g["q"], g["k"], g["v"], g["cum_gate"], g["beta"], g["do"],
                                  initial_state=g["h0"], d_final_state=g["dstate"])
    _close(res["o"], g["o"], 2e-5)
    _close(res["state"], g["state"], 2e-5)
    for name in ("dq", "dk", "dv", "dg", "dbeta", "dh0"):
        _close(res[name], g[name], 1e-4, 1e-3)


def test_chunk_packed_forward_and_grads(golden):
    g = golden("chunk_packed")
    res = orc.chunk_kda_grads_ref(g["q"], g["k"], g["v"], g["cum_gate"], g["beta"], g["do"],
                                  initial_state=g["h0"], d_final_state=g["dstate"],
                                  cu_seqlens=g["cu_seqlens"])
    _close(res["o"], g["o"], 2e-5)
    _close(res["state"], g["state"], 2e-5)
    assert torch.equal(res["state"][2].float(), g["h0"][2])
    for name in ("dq", "dk", "dv", "dg", "dbeta", "dh0"):
        _close(res[name], g[name], 1e-4, 1e-3)


def test_chunk_equals_recurrent_fp64():
    inp = orc.make_inputs(1, 150, 2, 32, 48, seed=3, with_state=True, dtype=torch.float64)
    h0 = inp["h0"].double()
    o_r, s_r = orc.recurrent_kda_ref(inp["q"], inp["k"], inp["v"], inp["gate_log2"].double(),
                                     inp["beta"].double(), h0)
    cum = orc.chunk_local_cumsum_ref(inp["gate_log2"].double(), 64)
    o_c, s_c = orc.chunk_kda_ref(inp["q"], inp["k"], inp["v"], cum, inp["beta"].double(), h0)
    torch.testing.assert_close(o_r, o_c, atol=1e-10, rtol=1e-8)
    torch.testing.assert_close(s_r, s_c, atol=1e-10, rtol=1e-8)


def test_config0(golden):
    """Benchmark configuration 0: B1 H4 T512 K=V=64 fp32, h0 = 0; inputs come from the seed."""
    g = golden("config0")
    inp = orc.make_inputs(1, 512, 4, 64, 64, seed=0)
    for n in ("q", "k", "v", "gate_log2", "beta"):
        s = torch.tensor([float(inp[n].double().sum()), float(inp[n].double().abs().sum())],
                         dtype=torch.float64)
        torch.testing.assert_close(s, g["sum_" + n], rtol=1e-9, atol=1e-9,
                                   msg=f"seeded input {n} drifted from the fixture's generator")
    o, st = orc.recurrent_kda_ref(inp["q"], inp["k"], inp["v"], inp["gate_log2"], inp["beta"])
    _close(o, g["o_recurrent"], 1e-6)
    _close(st, g["state_recurrent"], 1e-6)
    oc, sc = orc.chunk_kda_ref(inp["q"], inp["k"], inp["v"], inp["cum_gate"], inp["beta"])
    _close(oc[:, ::8], g["o_chunk_s8"], 2e-6)
    _close(sc, g["state_chunk"], 2e-6)
    # the natural-log statement of the configuration equals the log2 entry points on g*log2(e)
    _close(o[0, ::8], g["o_natural_fp64_s8"], 2e-6)
    _close(st[0], g["state_natural_fp64"], 2e-6)


def test_gate(golden):
    g = golden("gate")
    raw = g["raw"].bfloat16()
    fwd = orc.bounded_gate_cumsum_ref(raw, g["A_log"], g["dt_bias"])
    _close(fwd, g["fwd"], 1e-5)
    d_raw, dA, dbias = orc.bounded_gate_cumsum_bwd_ref(raw, g["A_log"], g["dt_bias"], g["dcum"])
    _close(d_raw, g["d_raw"], 1e-5)
    _close(dA, g["dA_log"], 1e-3)
    _close(dbias, g["d_dt_bias"], 1e-4)
    fwd_p = orc.bounded_gate_cumsum_ref(raw[:1, :131], g["A_log"], g["dt_bias"],
                                        cu_seqlens=g["cu_seqlens"])
    _close(fwd_p, g["fwd_packed"], 1e-5)
    _close(orc.chunk_local_cumsum_ref(g["dcum"], 16, reverse=True), g["revcumsum16"], 1e-5)


def test_l2norm(golden):
    g = golden("l2norm")
    y, rstd = orc.l2norm_ref(g["x"])
    _close(y, g["y"], 1e-6)
    _close(rstd, g["rstd"], 1e-5)
    _close(orc.l2norm_bwd_ref(g["y"], g["rstd"], g["dy"]), g["dx"], 1e-6)


def test_conv(golden):
    g = golden("conv")
    x = g["x"].clone().requires_grad_(True)
    w = g["w"].clone().requires_grad_(True)
    hist = g["hist"].clone().requires_grad_(True)
    # the oracle is plain differentiable torch, so its autograd gives the gradient oracle
    y, final = orc.causal_conv1d_ref(x, w, "silu", None, hist)
    _close(y, g["y"], 1e-5)
    _close(final, g["final"], 0)
    dx, dw, dh = torch.autograd.grad((y * g["dy"]).sum(), (x, w, hist))
    _close(dx, g["dx"], 1e-5)
    _close(dw, g["dw"], 1e-4)
    _close(dh, g["dhist"], 1e-5)


def test_slice_transition_composes():
    """h_out = M h_in + b: the context-parallel composition rule, against the recurrence."""
    inp = orc.make_inputs(1, 70, 2, 16, 24, seed=5, with_state=True, dtype=torch.float64)
    g2, beta, h0 = inp["gate_log2"].double(), inp["beta"].double(), inp["h0"].double()
    _, full = orc.recurrent_kda_ref(inp["q"], inp["k"], inp["v"], g2, beta, h0)
    _, zero = orc.recurrent_kda_ref(inp["q"], inp["k"], inp["v"], g2, beta, None)
    m = orc.slice_transition_ref(inp["k"][0], g2[0], beta[0])
    torch.testing.assert_close(full[0], m @ h0[0] + zero[0], atol=1e-12, rtol=1e-9)


def test_gated_output_norm_matches_torch_composition():
    """The epilogue oracle against the three torch operations the reference module applies
    (F.rms_norm, sigmoid, product) in fp64, values and gradients."""
    gen = torch.Generator().manual_seed(3)
    o = torch.randn(5, 7, 3, 128, generator=gen, dtype=torch.float64, requires_grad=True)
    z = torch.randn(5, 7, 3, 128, generator=gen, dtype=torch.float64, requires_grad=True)
    w = (1 + 0.1 * torch.randn(128, generator=gen, dtype=torch.float64)).requires_grad_()
    dy = torch.randn(5, 7, 3, 128, generator=gen, dtype=torch.float64)
    ref = torch.nn.functional.rms_norm(o, (128,), w, eps=1e-5) * z.sigmoid()
    got = orc.gated_output_norm_ref(o, z, w, 1e-5)
    _close(got, ref, 1e-12)
    for a, b in zip(torch.autograd.grad(got, (o, z, w), dy), torch.autograd.grad(ref, (o, z, w), dy)):
        _close(a, b, 1e-12)
