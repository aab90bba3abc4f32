"""The benchmark configurations at their full sizes, checked through size-independent properties:

* a batch row / packed sequence computed alone gives bitwise the same outputs and gradients
  (sequences are independent; the reference checks the same property at small sizes,
  test/test_kda_ragged_public_backward.py:142-191);
* a prefix computed alone gives bitwise the same outputs (causality);
* the output is linear in (v, initial state) for fixed q, k, gates and beta, and the backward pass
  is the adjoint of that linear map: <dO, o> + <dS, S_T> = <dv, v> + <dh0, h0> over all 8 x 4096 x 32
  (token, head) pairs at once;
* 1024 decode steps end in the state the chunked core reaches on the same tokens;
* the context-parallel boundary-state chain reproduces the single pass over 1 M tokens;

plus the fp32 CPU oracle on a slice small enough to finish in seconds.  Inputs are seeded synthetic
tensors with the shapes and distributions of the benchmark configurations, generated on the GPU.
"""

import pytest
import torch

import kda_b200
from kda_b200.dist import cp_chunk_forward
from oracle import kda_oracle as orc
from helpers import assert_budget, assert_normalised

pytestmark = pytest.mark.gpu
LOG2E = 1.4426950408889634
H, D = 32, 128


def _gen(seed):
    return torch.Generator(device="cuda").manual_seed(seed)


def _unit(shape, gen):
    x = torch.randn(shape, generator=gen, device="cuda")
    return (x / x.norm(dim=-1, keepdim=True)).bfloat16()


def _gate(shape, gen):
    """Per-token log2 gate, logsigmoid(N(0, 1)) / ln 2, fp32."""
    return torch.nn.functional.logsigmoid(torch.randn(shape, generator=gen, device="cuda")) * LOG2E


def _chunk_cumsum(g, offsets):
    """Chunk-local inclusive cumulative gate of packed sequences ([1, T, H, D], offsets on the host)."""
    out = torch.empty_like(g)
    for bos, eos in zip(offsets[:-1], offsets[1:]):
        n = eos - bos
        if n == 0:
            continue
        full = n // 64 * 64
        if full:
            out[0, bos:bos + full] = g[0, bos:bos + full].view(full // 64, 64, *g.shape[2:]).cumsum(1).view(
                full, *g.shape[2:])
        if n > full:
            out[0, bos + full:eos] = g[0, bos + full:eos].cumsum(0)
    return out


def _oracle_slice(q, k, v, g2, beta, h0, heads):
    """fp32 token recurrence on the CPU for a head slice of one sequence ([T, H, D] tensors)."""
    sl = slice(*heads)
    args = [t[None, :, sl].float().cpu() for t in (q, k, v, g2)]
    b = beta[None, :, sl].float().cpu()
    s0 = None if h0 is None else h0[None, sl].float().cpu()
    return orc.recurrent_kda_ref(*args, b, s0)


def test_config1_rows_are_independent_and_match_the_oracle():
    """B=8, T=4096, H=32, K=V=128, bf16 forward + backward."""
    torch.cuda.empty_cache()
    gen = _gen(101)
    B, T = 8, 4096
    q, k = _unit((B, T, H, D), gen), _unit((B, T, H, D), gen)
    v = torch.randn(B, T, H, D, generator=gen, device="cuda").bfloat16()
    g2 = _gate((B, T, H, D), gen)
    cum = g2.view(B, T // 64, 64, H, D).cumsum(2).view(B, T, H, D)
    beta = torch.sigmoid(torch.randn(B, T, H, generator=gen, device="cuda"))
    do = torch.randn(B, T, H, D, generator=gen, device="cuda").bfloat16()

    def run(rows):
        ins = [t[rows].detach().clone().requires_grad_(True) for t in (q, k, v, cum, beta)]
        o, _ = kda_b200.chunk_kda(*ins)
        return (o,) + torch.autograd.grad(o, ins, do[rows])

    full = run(slice(0, B))
    alone = run(slice(3, 4))
    for name, a, b in zip(("o", "dq", "dk", "dv", "dg", "dbeta"), full, alone):
        assert torch.equal(a[3:4], b), f"row 3 alone differs in {name}"
        assert torch.isfinite(a.float()).all(), name
    # causal: the first 512 tokens of row 3 against the fp32 recurrence, heads 5 and 6
    ro, _ = _oracle_slice(q[3, :512], k[3, :512], v[3, :512], g2[3, :512], beta[3, :512], None, (5, 7))
    assert_normalised(full[0][3, :512, 5:7].float(), ro[0], 2e-2, "config 1 output vs oracle")


def test_config1_linear_in_values_and_backward_is_the_adjoint():
    """B=8, T=4096, H=32: for fixed q, k, gates and beta the core is a linear map (v, h0) -> (o, S_T).
    Checked over the whole batch: additivity of the forward pass, and the inner-product identity
    <dO, o> + <dS, S_T> = <dv, v> + <dh0, h0> that ties the backward kernels (state-gradient walk and
    chunk backward) to the forward ones.  Every product is rounded to bf16 once on the way, so the
    two sides agree to about the bf16 spacing of the largest term, not bitwise."""
    torch.cuda.empty_cache()
    gen = _gen(131)
    B, T = 8, 4096
    q, k = _unit((B, T, H, D), gen), _unit((B, T, H, D), gen)
    va = torch.randn(B, T, H, D, generator=gen, device="cuda").bfloat16()
    vb = torch.randn(B, T, H, D, generator=gen, device="cuda").bfloat16()
    g2 = _gate((B, T, H, D), gen)
    cum = g2.view(B, T // 64, 64, H, D).cumsum(2).view(B, T, H, D)
    beta = torch.sigmoid(torch.randn(B, T, H, generator=gen, device="cuda"))
    ha = 0.05 * torch.randn(B, H, D, D, generator=gen, device="cuda")
    hb = 0.05 * torch.randn(B, H, D, D, generator=gen, device="cuda")
    do = torch.randn(B, T, H, D, generator=gen, device="cuda").bfloat16()
    dst = 0.1 * torch.randn(B, H, D, D, generator=gen, device="cuda")

    def fwd(v, h0):
        with torch.no_grad():
            return kda_b200.chunk_kda(q, k, v, cum, beta, h0, output_final_state=True)

    oa, sa = fwd(va, ha)
    ob, sb = fwd(vb, hb)
    # the summed values are rounded to bf16 once more (2^-9 relative), well inside the tolerance
    os_, ss = fwd((va.float() + vb.float()).bfloat16(), ha + hb)
    assert_normalised(os_.float(), oa.float() + ob.float(), 1e-2, "o(v_a + v_b) against o(v_a) + o(v_b)")
    assert_normalised(ss, sa + sb, 1e-2, "S_T(v_a + v_b) against S_T(v_a) + S_T(v_b)")
    del oa, sa, ob, sb, os_, ss

    ins = [t.detach().clone().requires_grad_(True) for t in (q, k, va, cum, beta, ha)]
    o, st = kda_b200.chunk_kda(*ins, output_final_state=True)
    grads = torch.autograd.grad((o, st), ins, (do, dst))
    dv, dh0 = grads[2], grads[5]
    lhs = (do.double() * o.double()).sum() + (dst.double() * st.double()).sum()
    rhs = (dv.double() * va.double()).sum() + (dh0.double() * ha.double()).sum()
    # scale of the sums: sqrt(number of terms) x typical term; bf16 rounding of o and dv gives a
    # relative 2^-9 on each term with random sign
    scale = ((do.double() * o.double()).abs().sum() + (dv.double() * va.double()).abs().sum()).item()
    assert abs(lhs.item() - rhs.item()) <= 2e-4 * scale, (lhs.item(), rhs.item(), scale)


def test_config2_packed_sequences_are_independent_and_match_the_oracle():
    """64 sequences, lengths uniform in [128, 8192], about 270 K packed tokens, int64 cu_seqlens,
    per-sequence h0 ~ N(0, 0.02), bf16 forward + backward with a final-state gradient."""
    torch.cuda.empty_cache()
    lengths = orc.draw_lengths(64, 128, 8192, seed=7)
    offsets = [0]
    for n in lengths:
        offsets.append(offsets[-1] + int(n))
    total = offsets[-1]
    gen = _gen(102)
    q, k = _unit((1, total, H, D), gen), _unit((1, total, H, D), gen)
    v = torch.randn(1, total, H, D, generator=gen, device="cuda").bfloat16()
    g2 = _gate((1, total, H, D), gen)
    cum = _chunk_cumsum(g2, offsets)
    beta = torch.sigmoid(torch.randn(1, total, H, generator=gen, device="cuda"))
    h0 = 0.02 * torch.randn(64, H, D, D, generator=gen, device="cuda")
    do = torch.randn(1, total, H, D, generator=gen, device="cuda").bfloat16()
    dst = torch.randn(64, H, D, D, generator=gen, device="cuda")
    cu = torch.tensor(offsets, dtype=torch.int64, device="cuda")

    ins = [t.detach().clone().requires_grad_(True) for t in (q, k, v, cum, beta, h0)]
    o, st = kda_b200.chunk_kda(*ins, cu_seqlens=cu, output_final_state=True)
    grads = torch.autograd.grad((o, st), ins, (do, dst))
    assert all(torch.isfinite(t.float()).all() for t in (o, st) + grads)

    shortest = min(range(64), key=lambda i: lengths[i])
    for i in sorted({0, 17, 63, shortest}):
        sl = slice(offsets[i], offsets[i + 1])
        one = [t[:, sl].detach().clone().requires_grad_(True) for t in (q, k, v, cum, beta)]
        one.append(h0[i:i + 1].detach().clone().requires_grad_(True))
        oo, ss = kda_b200.chunk_kda(*one, output_final_state=True)
        gg = torch.autograd.grad((oo, ss), one, (do[:, sl], dst[i:i + 1]))
        assert torch.equal(o[:, sl], oo), f"sequence {i}: output"
        assert torch.equal(st[i:i + 1], ss), f"sequence {i}: final state"
        for name, a, b in zip(("dq", "dk", "dv", "dg", "dbeta"), grads, gg):
            assert torch.equal(a[:, sl], b), f"sequence {i}: {name}"
        assert torch.equal(grads[5][i:i + 1], gg[5]), f"sequence {i}: dh0"
    sl = slice(offsets[shortest], offsets[shortest + 1])
    ro, rs = _oracle_slice(q[0, sl], k[0, sl], v[0, sl], g2[0, sl], beta[0, sl], h0[shortest], (0, 2))
    assert_normalised(o[0, sl, 0:2].float(), ro[0], 2e-2, "config 2 output vs oracle")
    assert_normalised(st[shortest, 0:2], rs[0], 2e-2, "config 2 final state vs oracle")


GRADS = ("dq", "dk", "dv", "dg", "dbeta", "dh0")


def _oracle_grads(q, k, v, cum, beta, h0, do, dst, heads):
    """fp64 gradients of one sequence ([T, H, D] tensors, `heads` a list of head indices) from the CPU
    oracle, plus the low-precision (bf16 intermediates) evaluation that sets the error budget."""
    def pick(t):
        return t[:, heads][None].float().cpu()

    args = [pick(t) for t in (q, k, v, cum)] + [beta[:, heads][None].float().cpu()]
    kw = dict(d_output=pick(do), initial_state=h0[heads][None].float().cpu(),
              d_final_state=dst[heads][None].float().cpu())
    gold = orc.chunk_kda_grads_ref(*args, dtype=torch.float64, **kw)
    low = orc.chunk_kda_grads_ref(*args, dtype=torch.float32, store_dtype=torch.bfloat16, **kw)
    return gold, low


def _check_against_oracle(got, gold, low, tag):
    for name in ("o", "state") + GRADS:
        assert_normalised(got[name].float(), gold[name].float(), 2e-2, f"{tag} {name}")
        assert_budget(got[name], gold[name], low[name], f"{tag} {name}")


def test_config1_backward_matches_the_oracle_over_a_64_chunk_chain():
    """Config-1 shape (T=4096, H=32): all six gradients, the output and the final state of two
    non-adjacent heads of the second batch row against the fp64 CPU oracle, with an initial state and
    a final-state cotangent, so the reverse state-gradient recurrence runs over the whole 64-chunk
    chain and the 64-bit (row, head) indexing is exercised
    (reference: test/test_kda_ragged_public_backward.py:142-273, test/test_kda_cute_forward.py:143-178)."""
    torch.cuda.empty_cache()
    gen = _gen(111)
    B, T = 2, 4096
    q, k = _unit((B, T, H, D), gen), _unit((B, T, H, D), gen)
    v = torch.randn(B, T, H, D, generator=gen, device="cuda").bfloat16()
    g2 = _gate((B, T, H, D), gen)
    cum = g2.view(B, T // 64, 64, H, D).cumsum(2).view(B, T, H, D)
    beta = torch.sigmoid(torch.randn(B, T, H, generator=gen, device="cuda"))
    h0 = 0.02 * torch.randn(B, H, D, D, generator=gen, device="cuda")
    do = torch.randn(B, T, H, D, generator=gen, device="cuda").bfloat16()
    dst = 0.1 * torch.randn(B, H, D, D, generator=gen, device="cuda")
    ins = [t.detach().clone().requires_grad_(True) for t in (q, k, v, cum, beta, h0)]
    o, st = kda_b200.chunk_kda(*ins, output_final_state=True)
    grads = torch.autograd.grad((o, st), ins, (do, dst))
    row, heads = 1, [5, 30]
    got = {"o": o[row][:, heads][None], "state": st[row, heads][None], "dh0": grads[5][row, heads][None]}
    for name, gr in zip(GRADS[:5], grads[:5]):
        got[name] = gr[row][:, heads][None]
    gold, low = _oracle_grads(q[row], k[row], v[row], cum[row], beta[row], h0[row], do[row], dst[row],
                              heads)
    _check_against_oracle(got, gold, low, "config 1")
    # the same step again gives the same bits (the dbeta and dg reductions have a fixed order)
    ins2 = [t.detach().clone().requires_grad_(True) for t in (q, k, v, cum, beta, h0)]
    o2, st2 = kda_b200.chunk_kda(*ins2, output_final_state=True)
    grads2 = torch.autograd.grad((o2, st2), ins2, (do, dst))
    assert torch.equal(o, o2) and torch.equal(st, st2)
    for name, a, b in zip(GRADS, grads, grads2):
        assert torch.equal(a, b), f"repeat run differs in {name}"


def test_config2_backward_matches_the_oracle_on_short_and_long_sequences():
    """The packed configuration (64 sequences of 128..8192 tokens, H=32, int64 offsets, initial states
    and final-state cotangents): the shortest sequence and one longer than 4096 tokens, two heads each,
    all gradients and dh0 against the fp64 CPU oracle."""
    torch.cuda.empty_cache()
    lengths = orc.draw_lengths(64, 128, 8192, seed=7)
    offsets = [0]
    for n in lengths:
        offsets.append(offsets[-1] + int(n))
    total = offsets[-1]
    gen = _gen(112)
    q, k = _unit((1, total, H, D), gen), _unit((1, total, H, D), gen)
    v = torch.randn(1, total, H, D, generator=gen, device="cuda").bfloat16()
    g2 = _gate((1, total, H, D), gen)
    cum = _chunk_cumsum(g2, offsets)
    beta = torch.sigmoid(torch.randn(1, total, H, generator=gen, device="cuda"))
    h0 = 0.02 * torch.randn(64, H, D, D, generator=gen, device="cuda")
    do = torch.randn(1, total, H, D, generator=gen, device="cuda").bfloat16()
    dst = 0.1 * torch.randn(64, H, D, D, generator=gen, device="cuda")
    cu = torch.tensor(offsets, dtype=torch.int64, device="cuda")
    ins = [t.detach().clone().requires_grad_(True) for t in (q, k, v, cum, beta, h0)]
    o, st = kda_b200.chunk_kda(*ins, cu_seqlens=cu, output_final_state=True)
    grads = torch.autograd.grad((o, st), ins, (do, dst))
    shortest = min(range(64), key=lambda i: lengths[i])
    longer = min((i for i in range(64) if lengths[i] > 4096), key=lambda i: lengths[i])
    for i, heads in ((shortest, [0, 31]), (longer, [7, 18])):
        sl = slice(offsets[i], offsets[i + 1])
        got = {"o": o[0, sl][:, heads][None], "state": st[i, heads][None],
               "dh0": grads[5][i, heads][None]}
        for name, gr in zip(GRADS[:5], grads[:5]):
            got[name] = gr[0, sl][:, heads][None]
        gold, low = _oracle_grads(q[0, sl], k[0, sl], v[0, sl], cum[0, sl], beta[0, sl], h0[i],
                                  do[0, sl], dst[i], heads)
        _check_against_oracle(got, gold, low, f"config 2 sequence {i} ({lengths[i]} tokens)")


def test_config3_1024_decode_steps():
    """256 sequences x H32, K=V=128, paged fp32 state, 1024 single-token steps with fresh bf16 tokens."""
    torch.cuda.empty_cache()
    n, steps = 256, 1024
    gen = _gen(103)
    q, k = _unit((n, steps, H, D), gen), _unit((n, steps, H, D), gen)
    v = torch.randn(n, steps, H, D, generator=gen, device="cuda").bfloat16()
    g2 = _gate((n, steps, H, D), gen).bfloat16()
    beta = torch.sigmoid(torch.randn(n, steps, H, generator=gen, device="cuda")).bfloat16()
    h0 = 0.02 * torch.randn(n, H, D, D, generator=gen, device="cuda")
    idx = torch.arange(1, n + 1, dtype=torch.int32, device="cuda")
    pool = torch.cat((torch.zeros_like(h0[:1]), h0), 0)          # slot 0 is the padding slot
    outs = torch.empty(n, steps, H, D, dtype=torch.bfloat16, device="cuda")
    for t in range(steps):
        outs[:, t:t + 1] = kda_b200.recurrent_kda(q[:, t:t + 1], k[:, t:t + 1], v[:, t:t + 1],
                                                  g2[:, t:t + 1], beta[:, t:t + 1], pool,
                                                  state_indices=idx)[0]
    assert torch.equal(pool[0], torch.zeros_like(pool[0])), "the padding slot was written"
    # the fp32 recurrence for sequence 7, heads 3 and 4, all 1024 steps
    ro, rs = _oracle_slice(q[7], k[7], v[7], g2[7].float(), beta[7].float(), h0[7], (3, 5))
    assert_normalised(outs[7, :, 3:5].float(), ro[0], 2e-2, "decode outputs vs oracle")
    assert_normalised(pool[8, 3:5], rs[0], 2e-3, "decode state vs oracle")
    # the chunked core on the same tokens ends in the same states
    cum = g2.float().view(n, steps // 64, 64, H, D).cumsum(2).view(n, steps, H, D)
    oc, sc = kda_b200.chunk_kda(q, k, v, cum, beta.float(), h0, output_final_state=True)
    assert_normalised(sc, pool[1:], 5e-2, "chunked core vs 1024 decode steps: state")
    assert_normalised(oc.float(), outs.float(), 5e-2, "chunked core vs 1024 decode steps: output")


def test_config4_one_million_tokens_prefix_and_context_parallel_chain():
    """B=1, T=1,048,576, H=32, K=V=128, bf16 forward: 64-bit offsets, 16384 chunks per head."""
    torch.cuda.empty_cache()
    T, piece = 1 << 20, 1 << 16
    gen = _gen(104)
    q = torch.empty(1, T, H, D, dtype=torch.bfloat16, device="cuda")
    k, v = torch.empty_like(q), torch.empty_like(q)
    cum = torch.empty(1, T, H, D, dtype=torch.float32, device="cuda")
    g_head = None
    for lo in range(0, T, piece):                       # piecewise, to bound fp32 temporaries
        q[0, lo:lo + piece] = _unit((piece, H, D), gen)
        k[0, lo:lo + piece] = _unit((piece, H, D), gen)
        v[0, lo:lo + piece] = torch.randn(piece, H, D, generator=gen, device="cuda").bfloat16()
        g2 = _gate((piece, H, D), gen)
        if lo == 0:
            g_head = g2[:2048].clone()
        cum[0, lo:lo + piece] = g2.view(piece // 64, 64, H, D).cumsum(1).view(piece, H, D)
        del g2
    beta = torch.sigmoid(torch.randn(1, T, H, generator=gen, device="cuda"))
    with torch.no_grad():
        o, st = kda_b200.chunk_kda(q, k, v, cum, beta, output_final_state=True)
        assert torch.isfinite(o.float()).all() and torch.isfinite(st).all()
        # causality at scale: the first 131072 tokens alone
        m = 1 << 17
        op, _ = kda_b200.chunk_kda(q[:, :m], k[:, :m], v[:, :m], cum[:, :m], beta[:, :m])
        assert torch.equal(o[:, :m], op), "prefix alone differs"
        del op
        ro, _ = _oracle_slice(q[0, :2048], k[0, :2048], v[0, :2048], g_head, beta[0, :2048], None, (0, 2))
        assert_normalised(o[0, :2048, 0:2].float(), ro[0], 2e-2, "config 4 output vs oracle")
        # the boundary-state chain of 8 contiguous slices, ranks run one after another
        world, per, mailbox, last_state = 8, T // 8, {}, None
        for rank in range(world):
            sl = slice(rank * per, (rank + 1) * per)

            def send(t, dst):
                mailbox[dst] = t.clone()

            def recv(t, src, rank=rank):
                t.copy_(mailbox.pop(rank))

            oc, last_state = cp_chunk_forward(q[:, sl], k[:, sl], v[:, sl], cum[:, sl], beta[:, sl],
                                              None, rank=rank, world=world, send=send, recv=recv)
            assert_normalised(oc.float(), o[:, sl].float(), 2e-2, f"slice {rank} output vs single pass")
            del oc
        assert_normalised(last_state, st, 2e-2, "chain final state vs single pass")
