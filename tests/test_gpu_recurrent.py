"""Recurrent scan / decode step parity (C ABI -> kda_recurrent_fwd) against the CPU oracle and the
golden vectors.  Tolerances follow the reference's decode tests
(test/test_kda_recurrent.py:74-98): 1e-5 for fp32 inputs, 2e-2 for 16-bit inputs."""

import pytest
import torch

import kda_b200
from oracle import kda_oracle as orc
from helpers import assert_normalised

pytestmark = pytest.mark.gpu


def test_golden_dense(golden):
    g = {k: v.cuda() for k, v in golden("recurrent_dense").items()}
    o, st = kda_b200.recurrent_kda(g["q"], g["k"], g["v"], g["gate"], g["beta"], g["h0"],
                                   output_final_state=True)
    torch.testing.assert_close(o, g["o"], atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(st, g["state"], atol=1e-5, rtol=1e-4)


def test_golden_packed(golden):
    g = {k: v.cuda() for k, v in golden("recurrent_packed").items()}
    o, st = kda_b200.recurrent_kda(g["q"], g["k"], g["v"], g["gate"], g["beta"], g["h0"],
                                   cu_seqlens=g["cu_seqlens"], output_final_state=True)
    torch.testing.assert_close(o, g["o"], atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(st, g["state"], atol=1e-5, rtol=1e-4)
    assert torch.equal(st[1], g["h0"][1])  # empty sequence: bitwise pass-through
    o64, _ = kda_b200.recurrent_kda(g["q"], g["k"], g["v"], g["gate"], g["beta"], g["h0"],
                                    cu_seqlens=g["cu_seqlens"].long())
    assert torch.equal(o64, o)  # int64 offsets are accepted


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2),
                                       (torch.float16, 2e-2)])
@pytest.mark.parametrize("kd,vd", [(128, 128), (64, 64), (24, 40), (256, 32)])
def test_scan_shapes(dtype, tol, kd, vd):
    inp = orc.make_inputs(2, 19, 3, kd, vd, seed=kd + vd, with_state=True)
    q, k, v, g = (inp[n].to(dtype) for n in ("q", "k", "v", "gate_log2"))
    beta = inp["beta"].to(dtype)
    ref_o, ref_s = orc.recurrent_kda_ref(q.float(), k.float(), v.float(), g.float(), beta.float(),
                                         inp["h0"])
    o, st = kda_b200.recurrent_kda(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(),
                                   inp["h0"].cuda(), output_final_state=True)
    assert o.dtype == dtype and st.dtype == torch.float32
    assert_normalised(o.float(), ref_o, tol, "output")
    assert_normalised(st, ref_s, tol, "state")


def test_config0_fp32(golden):
    """B1 H4 T512 K=V=64 fp32 through chunk_kda and recurrent_kda: <= 2e-3 max relative error."""
    g = golden("config0")
    inp = orc.make_inputs(1, 512, 4, 64, 64, seed=0)
    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    o, st = kda_b200.recurrent_kda(c["q"], c["k"], c["v"], c["gate_log2"], c["beta"],
                                   output_final_state=True)
    assert_normalised(o, g["o_recurrent"], 2e-3, "recurrent output")
    assert_normalised(st, g["state_recurrent"], 2e-3, "recurrent state")
    oc, sc = kda_b200.chunk_kda(c["q"], c["k"], c["v"], c["cum_gate"], c["beta"],
                                output_final_state=True)
    assert_normalised(oc, g["o_recurrent"], 2e-3, "chunk output")
    assert_normalised(sc, g["state_chunk"], 2e-3, "chunk state")
    big = g["o_recurrent"].abs() > 1e-2 * g["o_recurrent"].abs().max()
    rel = ((oc.cpu() - g["o_recurrent"]).abs() / g["o_recurrent"].abs())[big].max()
    assert rel <= 2e-3, f"max relative error {rel:.3e}"


def test_fp32_inputs_follow_the_reference_unless_exact_fp32_is_asked_for():
    """fp32 q, k, v at K = V = 128: the default rounds them to bf16 and runs the chunked kernels, with
    or without autograd, as the reference's fused path does (impl/fused.py:169-171);
    exact_fp32=True runs the fp32 token scan instead."""
    inp = orc.make_inputs(1, 130, 2, 128, 128, seed=13, with_state=True)
    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    args = (c["q"], c["k"], c["v"], c["cum_gate"], c["beta"], c["h0"])
    with torch.no_grad():
        o32, s32 = kda_b200.chunk_kda(*args, output_final_state=True)
        ob, sb = kda_b200.chunk_kda(c["q"].bfloat16(), c["k"].bfloat16(), c["v"].bfloat16(),
                                    *args[3:], output_final_state=True)
        oe, se = kda_b200.chunk_kda(*args, output_final_state=True, exact_fp32=True)
    assert o32.dtype == torch.float32 and torch.equal(o32, ob.float()) and torch.equal(s32, sb)
    leaves = [t.clone().requires_grad_() for t in args]
    og, sg = kda_b200.chunk_kda(*leaves, output_final_state=True)
    assert torch.equal(og, o32) and torch.equal(sg, s32), "train and eval numerics differ"
    ro, rs = orc.chunk_kda_ref(inp["q"], inp["k"], inp["v"], inp["cum_gate"], inp["beta"], inp["h0"])
    assert_normalised(oe, ro, 1e-5, "exact fp32 output")
    assert_normalised(se, rs, 1e-5, "exact fp32 state")
    with pytest.raises(ValueError):
        kda_b200.chunk_kda(*leaves, exact_fp32=True)


def test_decode_paged_pool():
    n, h, kd, vd, slots = 6, 2, 128, 128, 9
    inp = orc.make_inputs(n, 1, h, kd, vd, seed=9)
    gen = torch.Generator().manual_seed(5)
    pool = 0.02 * torch.randn(slots, h, kd, vd, generator=gen)
    idx = torch.tensor([3, -1, 5, 0, 8, 1], dtype=torch.int32)
    q, k, v, g = (inp[x].bfloat16() for x in ("q", "k", "v", "gate_log2"))
    beta = inp["beta"].bfloat16()
    pool_gpu = pool.cuda()
    o, none = kda_b200.recurrent_kda(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), pool_gpu,
                                     state_indices=idx.cuda())
    assert none is None
    for i, slot in enumerate(idx.tolist()):
        if slot <= 0:
            assert o[i].abs().max() == 0
            continue
        ro, rs = orc.recurrent_kda_ref(q[i:i + 1].float(), k[i:i + 1].float(), v[i:i + 1].float(),
                                       g[i:i + 1].float(), beta[i:i + 1].float(),
                                       pool[slot:slot + 1])
        assert_normalised(o[i].float(), ro[0], 2e-2, f"paged output {i}")
        assert_normalised(pool_gpu[slot], rs[0], 1e-4, f"paged state {i}")
    untouched = [s for s in range(slots) if s not in (3, 5, 8, 1)]
    assert torch.equal(pool_gpu[untouched].cpu(), pool[untouched])


@pytest.mark.parametrize("pad,n", [(2 * 128 * 128, 5), (64, 150), (2, 5)],
                         ids=["stride-2HKV", "stride+64", "stride+2"])
def test_decode_strided_paged_pool(pad, n):
    """A paged pool whose slots are contiguous inside but further apart than H*K*V elements (a view
    into a larger cache, as serving engines hand over; reference: test/test_kda_recurrent.py:56-71,
    207-290).  A slot stride that is a multiple of 128 takes the tensor-map decode kernel, the other
    two the token scan (with 300 (sequence, head) pairs its float4 form, with 10 its scalar form);
    the gaps between slots must stay untouched."""
    h, slots = 2, n + 2
    hkv = h * 128 * 128
    inp = orc.make_inputs(n, 1, h, 128, 128, seed=31)
    gen = torch.Generator().manual_seed(6)
    backing = 0.02 * torch.randn(slots, hkv + pad, generator=gen)
    backing_gpu = backing.cuda()
    pool_gpu = backing_gpu[:, :hkv].view(slots, h, 128, 128)
    assert pool_gpu.stride(0) == hkv + pad and not pool_gpu.is_contiguous()
    pool = backing[:, :hkv].reshape(slots, h, 128, 128)
    idx = (torch.randperm(slots - 1, generator=gen)[:n] + 1).to(torch.int32)
    idx[1], idx[4] = 0, -3                                   # padding rows
    q, k, v, g = (inp[x].bfloat16() for x in ("q", "k", "v", "gate_log2"))
    beta = inp["beta"].bfloat16()
    o, _ = kda_b200.recurrent_kda(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), pool_gpu,
                                  state_indices=idx.cuda())
    assert o[(idx <= 0).cuda()].abs().max() == 0
    live = idx[idx > 0].long()
    ro, rs = orc.recurrent_kda_ref(q[idx > 0].float(), k[idx > 0].float(), v[idx > 0].float(),
                                   g[idx > 0].float(), beta[idx > 0].float(), pool[live])
    assert_normalised(o[(idx > 0).cuda()].float(), ro, 2e-2, "strided pool outputs")
    assert_normalised(pool_gpu[live.cuda()], rs, 1e-4, "strided pool states")
    untouched = [s for s in range(slots) if s not in set(live.tolist())]
    assert torch.equal(pool_gpu[untouched].cpu(), pool[untouched])
    assert torch.equal(backing_gpu[:, hkv:].cpu(), backing[:, hkv:]), "the gaps between slots were written"


def test_decode_ring_many_items():
    """More (sequence, head) states than SMs: every persistent CTA walks several states through its
    shared-memory ring, with padding slots in between; three steps in a row on the same pool."""
    n, h, slots = 150, 4, 160
    gen = torch.Generator().manual_seed(11)
    pool = 0.02 * torch.randn(slots, h, 128, 128, generator=gen)
    idx = torch.randperm(slots - 1, generator=gen)[:n].to(torch.int32) + 1
    idx[::7] = 0                                            # padding rows
    pool_gpu, ref_pool = pool.cuda(), pool.clone()
    for step in range(3):
        inp = orc.make_inputs(n, 1, h, 128, 128, seed=20 + step)
        q, k, v, g = (inp[x].bfloat16() for x in ("q", "k", "v", "gate_log2"))
        beta = inp["beta"].bfloat16()
        o, _ = kda_b200.recurrent_kda(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), pool_gpu,
                                      state_indices=idx.cuda())
        live = (idx > 0).nonzero().flatten()
        sl = idx[live].long()
        ro, rs = orc.recurrent_kda_ref(q[live].float(), k[live].float(), v[live].float(),
                                       g[live].float(), beta[live].float(), ref_pool[sl])
        ref_pool[sl] = rs
        assert o[(idx <= 0).nonzero().flatten().cuda()].abs().max() == 0
        assert_normalised(o[live.cuda()].float(), ro, 2e-2, f"step {step} output")
        assert_normalised(pool_gpu[sl.cuda()], rs, 1e-4, f"step {step} state")
    spare = torch.ones(slots, dtype=torch.bool)
    spare[idx[idx > 0].long()] = False
    assert torch.equal(pool_gpu[spare.cuda()].cpu(), pool[spare])


def test_decode_steps_match_chunk_core():
    """64 decode steps == one chunk of the chunked core (reference: test_kda_recurrent.py:173-204)."""
    inp = orc.make_inputs(2, 64, 2, 128, 128, seed=4)
    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    q, k, v = (c[n].bfloat16() for n in ("q", "k", "v"))
    state = torch.zeros(2, 2, 128, 128, device="cuda")
    outs = []
    for t in range(64):
        o, state = kda_b200.recurrent_kda(q[:, t:t + 1], k[:, t:t + 1], v[:, t:t + 1],
                                          c["gate_log2"][:, t:t + 1], c["beta"][:, t:t + 1], state,
                                          output_final_state=True)
        outs.append(o)
    o_dec = torch.cat(outs, 1)
    o_chunk, s_chunk = kda_b200.chunk_kda(q, k, v, c["cum_gate"], c["beta"],
                                          output_final_state=True)
    assert_normalised(o_chunk.float(), o_dec.float(), 5e-2, "chunk vs decode output")
    assert_normalised(s_chunk, state, 5e-2, "chunk vs decode state")


def test_rejects_grad_and_bad_shapes():
    inp = orc.make_inputs(1, 4, 1, 16, 16, seed=1)
    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    with pytest.raises(RuntimeError):
        kda_b200.recurrent_kda(c["q"].requires_grad_(), c["k"], c["v"], c["gate_log2"], c["beta"])
    with pytest.raises(ValueError):
        kda_b200.recurrent_kda(c["q"].detach(), c["k"][:, :2], c["v"], c["gate_log2"], c["beta"])
    with pytest.raises(TypeError):
        kda_b200.recurrent_kda(c["q"].detach().double(), c["k"].double(), c["v"].double(),
                               c["gate_log2"].double(), c["beta"].double())


@pytest.mark.parametrize("dtype,tol,w", [(torch.bfloat16, 2e-2, 4), (torch.float16, 4e-3, 4),
                                         (torch.float32, 2e-3, 4), (torch.bfloat16, 2e-2, 2),
                                         (torch.bfloat16, 2e-2, 3), (torch.bfloat16, 2e-2, 5)])
def test_decode_step_fused_preprocessing(dtype, tol, w):
    """decode_step = conv decode + SiLU + l2norm(q, k) + bounded per-token gate + paged state update,
    against the composition of the CPU oracle's pieces; three steps on the same pools, with padding
    rows.  16-bit activations take the vector kernel, fp32 the scalar one; fp32 state."""
    from oracle.kda_oracle import (bounded_gate_cumsum_ref, causal_conv1d_ref, l2norm_ref,
                                   recurrent_kda_ref)

    n, h, slots = 20, 4, 24           # filter widths 2..4 take the vector kernel, wider ones the scalar one
    c = 3 * h * 128
    gen = torch.Generator().manual_seed(77)
    weight = (0.5 * torch.randn(c, w, generator=gen)).to(dtype)
    conv_state = torch.randn(slots, w - 1, c, generator=gen).to(dtype)
    pool = 0.02 * torch.randn(slots, h, 128, 128, generator=gen)
    a_log = 0.3 * torch.randn(h, generator=gen)
    dt_bias = 0.3 * torch.randn(h, 128, generator=gen)
    idx = torch.randperm(slots - 1, generator=gen)[:n].to(torch.int32) + 1
    idx[3], idx[11] = 0, -1                                   # padding rows
    live = (idx > 0).nonzero().flatten()
    sl = idx[live].long()
    conv_gpu, pool_gpu = conv_state.cuda(), pool.cuda()
    conv_ref, pool_ref = conv_state.clone(), pool.clone()
    for step in range(3):
        x = torch.randn(n, c, generator=gen).to(dtype)
        raw = torch.randn(n, h, 128, generator=gen).to(dtype)
        beta = torch.sigmoid(torch.randn(n, h, generator=gen)).to(dtype)
        o = kda_b200.decode_step(x.cuda(), weight.cuda(), conv_gpu, raw.cuda(), a_log.cuda(),
                                 dt_bias.cuda(), beta.cuda(), pool_gpu, idx.cuda())
        # oracle: each piece in fp32 on the bf16-rounded inputs
        y, hist = causal_conv1d_ref(x[live, None].float(), weight.float(), activation="silu",
                                    initial_state=conv_ref[sl].float())
        conv_ref[sl] = hist.to(dtype)
        y = y[:, 0].view(-1, 3, h, 128)
        q, k, v = l2norm_ref(y[:, 0])[0], l2norm_ref(y[:, 1])[0], y[:, 2]
        g = bounded_gate_cumsum_ref(raw[live, None].float(), a_log, dt_bias, chunk_size=1)
        # the kernel hands bf16 q, k, v to the state update
        q, k, v = (t.to(dtype).float()[:, None] for t in (q, k, v))
        ro, rs = recurrent_kda_ref(q, k, v, g, beta[live, None].float(), pool_ref[sl])
        pool_ref[sl] = rs
        assert o[(idx <= 0).nonzero().flatten().cuda()].abs().max() == 0
        assert_normalised(o[live.cuda()].float(), ro[:, 0], tol, f"step {step} output")
        assert_normalised(pool_gpu[sl.cuda()], rs, tol, f"step {step} state")
        assert torch.equal(conv_gpu[sl.cuda()].cpu(), conv_ref[sl]), f"step {step} conv history"
    spare = torch.ones(slots, dtype=torch.bool)
    spare[sl] = False
    assert torch.equal(pool_gpu[spare.cuda()].cpu(), pool[spare])
    assert torch.equal(conv_gpu[spare.cuda()].cpu(), conv_state[spare])
