"""The operators run on the caller's stream without host synchronisation, read packed-sequence
offsets on the device, and size their grids by the chunk capacity -- so a captured CUDA graph can be
replayed on new data and on a different split of the same number of tokens into sequences (the
reference's fixed-capacity graph replay, attn_gym/linear/kda/chunk_scheduler.py:112-239)."""

import pytest
import torch

import kda_b200
from helpers import assert_normalised
from oracle import kda_oracle as orc

pytestmark = pytest.mark.gpu


def _packed_case(lengths, heads, seed):
    total = sum(lengths)
    inp = orc.make_inputs(1, total, heads, 128, 128, seed=seed)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    g = orc.chunk_local_cumsum_ref(inp["gate_log2"], 64, cu_seqlens=cu)
    gen = torch.Generator().manual_seed(seed + 1)
    return {"q": inp["q"].bfloat16(), "k": inp["k"].bfloat16(), "v": inp["v"].bfloat16(), "g": g,
            "beta": inp["beta"], "do": torch.randn(inp["v"].shape, generator=gen).bfloat16(), "cu": cu}


def _step(bufs):
    leaves = [bufs[n].detach().requires_grad_() for n in ("q", "k", "v", "g", "beta")]
    o, _ = kda_b200.chunk_kda(*leaves, cu_seqlens=bufs["cu"])
    grads = torch.autograd.grad(o, leaves, bufs["do"])
    return (o,) + tuple(grads)


def test_packed_forward_backward_graph_replays_on_other_sequences():
    first = _packed_case([200, 333, 64, 427], 2, seed=51)       # 1024 tokens, 4 sequences
    second = _packed_case([5, 700, 130, 189], 2, seed=52)       # same token count, different split
    static = {n: t.cuda().clone() for n, t in first.items()}
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):                               # warm-up outside the capture
        for _ in range(2):
            _step(static)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = _step(static)
    for case in (second, first):
        for n, t in case.items():
            static[n].copy_(t)
        graph.replay()
        torch.cuda.synchronize()
        got = [t.clone() for t in outs]
        want = _step({n: t.cuda() for n, t in case.items()})
        for name, a, b in zip(("o", "dq", "dk", "dv", "dg", "dbeta"), got, want):
            assert torch.equal(a, b), f"graph replay differs from the eager call: {name}"
    # and against the oracle, for the second split
    for n, t in second.items():
        static[n].copy_(t)
    graph.replay()
    ref = orc.chunk_kda_ref(second["q"].float(), second["k"].float(), second["v"].float(),
                            second["g"], second["beta"], cu_seqlens=second["cu"])[0]
    assert_normalised(outs[0].float(), ref, 2e-2, "replayed output vs oracle")


def test_decode_step_graph_replay():
    n, h, slots = 16, 4, 20
    c = 3 * h * 128
    gen = torch.Generator().manual_seed(61)
    weight = (0.5 * torch.randn(c, 4, generator=gen)).bfloat16().cuda()
    a_log = (0.3 * torch.randn(h, generator=gen)).cuda()
    dt_bias = (0.3 * torch.randn(h, 128, generator=gen)).cuda()
    conv0 = torch.randn(slots, 3, c, generator=gen).bfloat16().cuda()
    pool0 = (0.02 * torch.randn(slots, h, 128, 128, generator=gen)).cuda()
    idx = (torch.randperm(slots - 1, generator=gen)[:n].to(torch.int32) + 1).cuda()
    steps = [(torch.randn(n, c, generator=gen).bfloat16().cuda(),
              torch.randn(n, h, 128, generator=gen).bfloat16().cuda(),
              torch.sigmoid(torch.randn(n, h, generator=gen)).bfloat16().cuda()) for _ in range(3)]

    conv_e, pool_e = conv0.clone(), pool0.clone()
    eager = [kda_b200.decode_step(x, weight, conv_e, raw, a_log, dt_bias, beta, pool_e, idx).clone()
             for x, raw, beta in steps]

    conv_g, pool_g = conv0.clone(), pool0.clone()
    sx, sraw, sbeta = (t.clone() for t in steps[0])
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        kda_b200.decode_step(sx, weight, conv_g, sraw, a_log, dt_bias, sbeta, pool_g, idx)
    torch.cuda.current_stream().wait_stream(side)
    conv_g.copy_(conv0), pool_g.copy_(pool0)                    # undo the warm-up step
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = kda_b200.decode_step(sx, weight, conv_g, sraw, a_log, dt_bias, sbeta, pool_g, idx)
    conv_g.copy_(conv0), pool_g.copy_(pool0)                    # capture does not execute
    for (x, raw, beta), want in zip(steps, eager):
        sx.copy_(x), sraw.copy_(raw), sbeta.copy_(beta)
        graph.replay()
        assert torch.equal(out, want)
    assert torch.equal(conv_g, conv_e) and torch.equal(pool_g, pool_e)
