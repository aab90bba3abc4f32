"""Context-parallel forward on the CUDA kernels: the ranks of the boundary-state chain are run one
after another in this process (mailbox send/recv), which exercises kda_chunk_fwd_prepare,
kda_chunk_fwd_state (zero state, identity/transition, true state) and kda_state_affine.  The
result must equal the single-GPU chunked forward of the whole sequence."""

import pytest
import torch

import kda_b200
from kda_b200.dist import CudaSlice, cp_chunk_forward
from oracle import kda_oracle as orc
from helpers import assert_normalised

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4])
def test_cp_matches_single_gpu(world):
    per = 128
    total = per * world + 50
    inp = orc.make_inputs(1, total, 2, 128, 128, seed=31, with_state=True)
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
                     c["beta"])
    m = part.transition()
    ref = orc.slice_transition_ref(inp["k"][0].bfloat16().float(), inp["gate_log2"][0],
                                   inp["beta"][0])
    assert_normalised(m[0], ref, 2e-2, "slice transition")


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
