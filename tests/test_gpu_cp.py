"""Context-parallel forward on the CUDA kernels: the ranks of the boundary-state chain are run one
after another in this process (mailbox send/recv), which exercises kda_chunk_fwd_prepare,
kda_chunk_slice_map (zero-state walk + transition walk with its measured early exit),
kda_chunk_fwd_state (true state, chunk-limited) and kda_state_affine.  The result must equal the
single-GPU chunked forward of the whole sequence."""

import pytest
import torch

import kda_b200
from kda_b200.dist import CudaSlice, cp_chunk_forward
from oracle import kda_oracle as orc
from helpers import assert_normalised, to_cuda

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("gate_scale", [1.0, 0.02], ids=["forgetful-gates", "mild-gates"])
@pytest.mark.parametrize("world,per", [(2, 128), (4, 128), (2, 1024)])
def test_cp_matches_single_gpu(world, per, gate_scale):
    """With the benchmark's gates (logsigmoid of N(0, 1), about 2^-74 per chunk) a slice forgets its
    entering state within a few chunks and the corrective pass is cut short; with gates scaled by
    0.02 the transition stays dense and every chunk is redone.  Both must match the single pass."""
    total = per * world + 50
    inp = orc.make_inputs(1, total, 2, 128, 128, seed=31, with_state=True)
    inp["cum_gate"] = inp["cum_gate"] * gate_scale
    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    q, k, v = (c[n].bfloat16() for n in ("q", "k", "v"))
    full_o, full_s = kda_b200.chunk_kda(q, k, v, c["cum_gate"], c["beta"], c["h0"],
                                        output_final_state=True)
    mailbox = {}
    outs, last_state = [], None
    for rank in range(world):
        lo = per * rank
        hi = total if rank + 1 == world else lo + per
        sl = slice(lo, hi)

        def send(t, dst):
            mailbox[dst] = t.clone()

        def recv(t, src, rank=rank):
            t.copy_(mailbox.pop(rank))

        o, s = cp_chunk_forward(q[:, sl], k[:, sl], v[:, sl], c["cum_gate"][:, sl], c["beta"][:, sl],
                                c["h0"], rank=rank, world=world, send=send, recv=recv)
        outs.append(o)
        last_state = s
    out = torch.cat(outs, 1)
    assert_normalised(out.float(), full_o.float(), 2e-2, "cp output vs single GPU")
    assert_normalised(last_state, full_s, 2e-2, "cp final state vs single GPU")
    ref_o, ref_s = orc.chunk_kda_ref(q.float().cpu(), k.float().cpu(), v.float().cpu(),
                                     inp["cum_gate"], inp["beta"], inp["h0"])
    assert_normalised(out.float(), ref_o, 2e-2, "cp output vs oracle")
    assert_normalised(last_state, ref_s, 2e-2, "cp final state vs oracle")


def test_transition_matches_oracle():
    inp = orc.make_inputs(1, 128, 2, 128, 128, seed=32)
    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    part = CudaSlice(c["q"].bfloat16(), c["k"].bfloat16(), c["v"].bfloat16(), c["cum_gate"],
                     c["beta"], segments=1)
    m = part.transition()
    ref = orc.slice_transition_ref(inp["k"][0].bfloat16().float(), inp["gate_log2"][0],
                                   inp["beta"][0])
    assert_normalised(m[0], ref, 2e-2, "slice transition")


def test_slice_map_in_one_launch_equals_the_two_passes():
    """kda_chunk_slice_map gives b (zero entering state) and the transition M in one launch; both are
    bitwise what the two separate state passes give.  Mild gates, so that M is far from zero."""
    inp = orc.make_inputs(1, 192, 2, 128, 128, seed=34)
    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    cum = 0.02 * c["cum_gate"]
    part = CudaSlice(c["q"].bfloat16(), c["k"].bfloat16(), c["v"].bfloat16(), cum, c["beta"], segments=1)
    out, b, m, limit = part.slice_map()
    assert torch.equal(b, part.zero_state_result())
    assert torch.equal(m, part.transition())
    assert torch.equal(out, part.run(None)[0])
    assert float(m.abs().max()) > 1e-2
    assert limit.tolist() == [[3, 3]], "a dense transition must not cut the corrective pass"
    ref = orc.slice_transition_ref(inp["k"][0].bfloat16().float(), 0.02 * inp["gate_log2"][0],
                                   inp["beta"][0])
    assert_normalised(m[0], ref, 2e-2, "slice transition (mild gates)")


def test_forgetful_gates_cut_the_corrective_pass_short():
    """Benchmark gates over 32 chunks: the transition walk reports that the slice forgets its entering
    state after a few chunks; M is then exactly zero, and the chunk-limited corrective pass gives what
    the full pass with the true entering state gives."""
    inp = orc.make_inputs(1, 2048, 2, 128, 128, seed=35, with_state=True)
    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    part = CudaSlice(c["q"].bfloat16(), c["k"].bfloat16(), c["v"].bfloat16(), c["cum_gate"], c["beta"],
                     segments=1)
    h_in = 50.0 * c["h0"]
    out, b, m, limit = part.slice_map()
    assert int(limit.max()) < 32 and int(limit.min()) >= 1, limit.tolist()
    assert float(m.abs().max()) == 0.0
    full_o, full_s = part.run(h_in)
    fixed = part.correct(out.clone(), h_in, limit)
    assert_normalised(fixed.float(), full_o.float(), 1e-4, "chunk-limited corrective pass vs full pass")
    assert not torch.equal(out, full_o), "the entering state must matter in the leading chunks"
    assert_normalised(part.affine(m, h_in, b), full_s, 1e-6, "M h_in + b vs the full pass")
    from kda_b200 import _cabi
    assert _cabi.lib().kda_device_error_word() == 0


@pytest.mark.parametrize("gate_scale", [1.0, 0.02], ids=["forgetful-gates", "mild-gates"])
@pytest.mark.parametrize("segments", [2, 3])
def test_a_slice_walked_in_segments_has_the_same_affine_map(segments, gate_scale):
    """A slice cut into segments that are walked in parallel: the composed (b, M), the outputs and the
    leaving state for a given entering state agree with the serial walk of the slice."""
    inp = orc.make_inputs(1, 64 * 12 + 30, 2, 128, 128, seed=36, with_state=True)
    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    cum = gate_scale * c["cum_gate"]
    args = (c["q"].bfloat16(), c["k"].bfloat16(), c["v"].bfloat16(), cum, c["beta"])
    h_in = 30.0 * c["h0"]
    serial, split = CudaSlice(*args, segments=1), CudaSlice(*args, segments=segments)
    assert split.segs == segments and split.nseq == segments
    so, sb, sm, _ = serial.slice_map()
    po, pb, pm, limit = split.slice_map()
    tol = 1e-4 if gate_scale == 1.0 else 1e-2
    assert_normalised(pb, sb, tol, "composed b")
    if gate_scale != 1.0:
        assert_normalised(pm, sm, tol, "composed M")
    else:
        assert float(pm.abs().max()) == 0.0 and float(sm.abs().max()) == 0.0
    ref_o, ref_s = serial.run(h_in)
    got_o, got_s = split.run(h_in)
    assert_normalised(got_o.float(), ref_o.float(), tol, "outputs of the segmented walk")
    assert_normalised(got_s, ref_s, tol, "leaving state of the segmented walk")


@pytest.mark.parametrize("world", [2, 3])
def test_cp_backward_matches_single_gpu(world):
    """The state-gradient chain (ranks run one after another, last rank first) against the backward
    of the unsplit sequence on one GPU."""
    from kda_b200.dist import _cp_forward, cp_chunk_backward

    per = 128
    total = per * world + 50
    inp = orc.make_inputs(1, total, 2, 128, 128, seed=33, with_state=True)
    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    gen = torch.Generator().manual_seed(6)
    d_out = torch.randn(inp["v"].shape, generator=gen).bfloat16().cuda()
    d_final = torch.randn(inp["h0"].shape, generator=gen).cuda()
    names = ("q", "k", "v", "cum_gate", "beta", "h0")
    leaves = [(c[n].bfloat16() if n in ("q", "k", "v") else c[n]).clone().requires_grad_() for n in names]
    o, s = kda_b200.chunk_kda(*leaves, output_final_state=True)
    ref = torch.autograd.grad((o, s), leaves, (d_out, d_final))

    mailbox = {}

    def send(t, dst):
        mailbox[dst] = t.clone()

    def make_recv(rank):
        def recv(t, src):
            t.copy_(mailbox.pop(rank))
        return recv

    def args_of(rank):
        sl = slice(per * rank, total if rank + 1 == world else per * (rank + 1))
        return sl, [leaves[i].detach()[:, sl] for i in range(5)]

    kept = {}
    for rank in range(world):
        sl, args = args_of(rank)
        kept[rank] = _cp_forward(*args, c["h0"], rank=rank, world=world, send=send,
                                 recv=make_recv(rank))[2:]
    grads = {}
    for rank in reversed(range(world)):
        sl, args = args_of(rank)
        h_in, trans = kept[rank]
        grads[rank] = cp_chunk_backward(*args, h_in, trans, d_out[:, sl],
                                        d_final if rank + 1 == world else None, rank=rank,
                                        world=world, send=send, recv=make_recv(rank))
    for i, name in enumerate(("dq", "dk", "dv", "d_gate", "d_beta")):
        got = torch.cat([grads[r][i] for r in range(world)], 1)
        assert_normalised(got.float(), ref[i].float(), 2e-2, f"cp {name} vs single GPU")
    assert_normalised(grads[0][5], ref[5], 2e-2, "cp d_initial_state vs single GPU")


def test_state_gradient_walk_alone_equals_the_full_backward():
    """The reverse state walk on kept intermediates (what a middle rank of the backward chain runs
    before the next slice's state gradient has arrived) returns the entering-state gradient of the
    full backward pass bit for bit, leaves the intermediates intact, and the full backward pass on
    the same buffer afterwards equals autograd on a fresh forward pass."""
    from kda_b200.dist import CudaSliceTape, cuda_slice_grads

    inp = to_cuda(orc.make_inputs(2, 200, 2, 128, 128, seed=31), torch.bfloat16)
    gen = torch.Generator(device="cuda").manual_seed(5)
    h_in = 0.1 * torch.randn(2, 2, 128, 128, generator=gen, device="cuda")
    d_out = torch.randn(2, 200, 2, 128, generator=gen, device="cuda").bfloat16()
    dh_out = 0.1 * torch.randn(2, 2, 128, 128, generator=gen, device="cuda")
    args = (inp["q"], inp["k"], inp["v"], inp["cum_gate"], inp["beta"])
    ref = cuda_slice_grads(*args, h_in, d_out, dh_out)
    ref0 = cuda_slice_grads(*args, h_in, d_out, torch.zeros_like(dh_out))
    tape = CudaSliceTape(*args, h_in)
    assert torch.equal(tape.state_grad(d_out, torch.zeros_like(dh_out)), ref0[5])
    assert torch.equal(tape.state_grad(d_out, dh_out), ref[5])
    for name, a, b in zip(("dq", "dk", "dv", "dg", "dbeta", "dh_in"), tape.grads(d_out, dh_out), ref):
        assert torch.equal(a, b), name
