"""Chunked forward / backward parity of the bf16 K=V=128 kernels (C ABI: kda_chunk_fwd / kda_chunk_bwd)
against the fp32 CPU oracle evaluated on the same bf16-rounded inputs.

Tolerance (stated by the task): <= 2e-2 max abs error on normalised outputs, gradients and final
states for bf16 inputs, against an fp32 reference.
"""

import pytest
import torch

import kda_b200
from oracle import kda_oracle as orc
from helpers import assert_normalised, norm_err

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _case(batch, tokens, heads, seed, lengths=None, with_state=True):
    inp = orc.make_inputs(batch, tokens, heads, 128, 128, seed=seed, with_state=with_state,
                          lengths=lengths)
    for n in ("q", "k", "v"):
        inp[n] = inp[n].bfloat16()
    return inp


def _run_fused(inp, do=None, dst=None, grad=False, recompute=False):
    q, k, v = (inp[n].cuda().requires_grad_(grad) for n in ("q", "k", "v"))
    g = inp["cum_gate"].cuda().requires_grad_(grad)
    beta = inp["beta"].cuda().requires_grad_(grad)
    h0 = None if inp["h0"] is None else inp["h0"].cuda().requires_grad_(grad)
    cu = None if inp["cu_seqlens"] is None else inp["cu_seqlens"].cuda()
    o, st = kda_b200.chunk_kda(q, k, v, g, beta, h0, cu_seqlens=cu, output_final_state=True,
                               recompute=recompute)
    res = {"o": o, "state": st}
    if grad:
        loss = (o.float() * do.cuda()).sum()
        if dst is not None:
            loss = loss + (st * dst.cuda()).sum()
        wrt = [q, k, v, g, beta] + ([h0] if h0 is not None else [])
        grads = torch.autograd.grad(loss, wrt)
        for name, gr in zip(["dq", "dk", "dv", "dg", "dbeta", "dh0"], grads):
            res[name] = gr
    return res


def _active(inp, x):
    """Slice a [1, T, ...] tensor of a packed case to its active prefix."""
    if inp["cu_seqlens"] is None:
        return x
    return x[:, : int(inp["cu_seqlens"][-1])]


CASES = [
    dict(batch=1, tokens=64, heads=1, seed=1),
    dict(batch=2, tokens=256, heads=2, seed=2),
    dict(batch=1, tokens=130, heads=2, seed=3),                       # partial tail chunk
    dict(batch=3, tokens=100, heads=1, seed=4),                       # dense rows not chunk aligned
    dict(batch=1, tokens=300, heads=2, seed=5, lengths=[65, 63, 0, 30, 128]),
    dict(batch=1, tokens=200, heads=1, seed=6, lengths=[0, 1, 64, 0, 65]),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"B{c['batch']}T{c['tokens']}H{c['heads']}")
def test_forward(case):
    inp = _case(**case)
    res = _run_fused(inp)
    ref_o, ref_s = orc.chunk_kda_ref(inp["q"].float(), inp["k"].float(), inp["v"].float(),
                                     inp["cum_gate"], inp["beta"], inp["h0"], inp["cu_seqlens"])
    assert res["o"].dtype == torch.bfloat16 and res["state"].dtype == torch.float32
    assert_normalised(_active(inp, res["o"]).float(), _active(inp, ref_o), TOL, "output")
    assert_normalised(res["state"], ref_s, TOL, "final state")
    if inp["cu_seqlens"] is not None:
        lens = inp["cu_seqlens"][1:] - inp["cu_seqlens"][:-1]
        for s in (lens == 0).nonzero().flatten().tolist():
            assert torch.equal(res["state"][s].cpu(), inp["h0"][s]), "empty sequence state"


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"B{c['batch']}T{c['tokens']}H{c['heads']}")
def test_backward(case):
    inp = _case(**case)
    gen = torch.Generator().manual_seed(100 + case["seed"])
    do = torch.randn(inp["v"].shape, generator=gen).bfloat16().float()
    nseq = case["batch"] if inp["cu_seqlens"] is None else inp["cu_seqlens"].numel() - 1
    dst = 0.1 * torch.randn(nseq, case["heads"], 128, 128, generator=gen)
    if inp["cu_seqlens"] is not None:
        do[:, int(inp["cu_seqlens"][-1]):] = 0
    res = _run_fused(inp, do, dst, grad=True)
    ref = orc.chunk_kda_grads_ref(inp["q"].float(), inp["k"].float(), inp["v"].float(),
                                  inp["cum_gate"], inp["beta"], do, inp["h0"], dst,
                                  inp["cu_seqlens"], dtype=torch.float32)
    report = {n: norm_err(_active(inp, res[n]).float() if n != "dh0" else res[n],
                          _active(inp, ref[n]) if n != "dh0" else ref[n])
              for n in ("dq", "dk", "dv", "dg", "dbeta", "dh0")}
    print("normalised gradient errors:", {k: f"{v:.2e}" for k, v in report.items()})
    for name, err in report.items():
        assert err <= TOL, f"{name}: normalised max error {err:.3e} > {TOL}"
    if inp["cu_seqlens"] is not None:
        lens = inp["cu_seqlens"][1:] - inp["cu_seqlens"][:-1]
        for s in (lens == 0).nonzero().flatten().tolist():
            assert torch.equal(res["dh0"][s].cpu(), dst[s]), "empty sequence state gradient"


@pytest.mark.parametrize("case", [CASES[1], CASES[4]], ids=["dense", "packed"])
def test_kept_intermediates_equal_recompute(case):
    """The default training path keeps the forward intermediates; recompute=True rebuilds them in
    the backward pass as the reference does (bwd/cute/chunk_kda_bwd.py:54-85).  Same kernels on
    the same values: every result is bitwise equal."""
    inp = _case(**case)
    gen = torch.Generator().manual_seed(99)
    do = torch.randn(inp["v"].shape, generator=gen)
    dst = torch.randn(inp["h0"].shape, generator=gen)
    kept = _run_fused(inp, do, dst, grad=True)
    again = _run_fused(inp, do, dst, grad=True, recompute=True)
    for name in kept:
        assert torch.equal(kept[name], again[name]), name


@pytest.mark.parametrize("case", [CASES[1], CASES[4]], ids=["dense", "packed"])
@pytest.mark.parametrize("recompute", [False, True], ids=["kept", "recompute"])
def test_value_split_of_the_state_recurrence_gives_the_same_bits(case, recompute):
    """The serial state kernels run 1, 2 or 4 CTAs per (sequence, head), each owning a slice of the
    value columns (the reference tiles the same dimension: fwd/triton/chunk_delta_h.py:166,
    bwd/cute/chunk_delta_h_bwd_v1_dispatch.py:53-55).  The products are separable along v, so
    outputs, states and all gradients are bitwise the same for every split."""
    from kda_b200 import _cabi

    inp = _case(**case)
    gen = torch.Generator().manual_seed(98)
    do = torch.randn(inp["v"].shape, generator=gen)
    dst = torch.randn(inp["h0"].shape, generator=gen)
    lib = _cabi.lib()
    runs = {}
    try:
        for split in (1, 2, 4):
            assert lib.kda_set_state_value_split(split) == 0
            runs[split] = _run_fused(inp, do, dst, grad=True, recompute=recompute)
    finally:
        lib.kda_set_state_value_split(0)
    assert lib.kda_set_state_value_split(3) == -1
    for split in (2, 4):
        for name in runs[1]:
            assert torch.equal(runs[1][name], runs[split][name]), f"split {split}: {name}"
    assert lib.kda_device_error_word() == 0


@pytest.mark.parametrize("gate_scale", [1.0, 0.02], ids=["forgetful-gates", "mild-gates"])
@pytest.mark.parametrize("segments", [2, 3, 5])
def test_rows_walked_in_parallel_segments_match_the_serial_walk(segments, gate_scale):
    """Long rows of a small dense batch are cut into segments that are walked in parallel and
    stitched by the affine boundary-state map (kda_chunk_fwd_dense).  Forced here on a short case:
    outputs, final states and -- through the kept h[c] / v_new -- all gradients must agree with the
    serial walk to the resolution of the fp32 state, for gates that forget within a few chunks (the
    corrective pass is cut short) and for gates that never do (it redoes every chunk)."""
    from kda_b200 import _cabi

    inp = _case(2, 64 * 23 + 17, 2, seed=21)          # 24 chunks per row, partial tail
    inp["cum_gate"] = inp["cum_gate"] * gate_scale
    inp["h0"] = 20.0 * inp["h0"]
    gen = torch.Generator().manual_seed(97)
    do = torch.randn(inp["v"].shape, generator=gen)
    dst = torch.randn(inp["h0"].shape, generator=gen)
    lib = _cabi.lib()
    serial = _run_fused(inp, do, dst, grad=True)
    try:
        assert lib.kda_set_row_segments(segments) == 0
        split = _run_fused(inp, do, dst, grad=True)
        plain = _run_fused(inp)                         # the forward-only entry point as well
    finally:
        lib.kda_set_row_segments(0)
    # gates that forget: the corrective pass restores the serial walk's bits almost everywhere;
    # gates that do not: the boundary states come from M h_in + b, whose bf16 product roundings differ
    # from the serial walk's, so the two agree like two bf16 evaluations do
    tol = 1e-4 if gate_scale == 1.0 else 1e-2
    for name in serial:
        assert_normalised(split[name].float(), serial[name].float(), tol, f"{segments} segments: {name}")
    assert torch.equal(plain["o"], split["o"]) and torch.equal(plain["state"], split["state"])
    ref = orc.chunk_kda_grads_ref(inp["q"].float(), inp["k"].float(), inp["v"].float(), inp["cum_gate"],
                                  inp["beta"], do.bfloat16().float(), inp["h0"], dst, dtype=torch.float32)
    for name in serial:
        assert_normalised(split[name].float(), ref[name], TOL, f"{segments} segments: {name} vs oracle")
    assert lib.kda_device_error_word() == 0


@pytest.mark.parametrize("case", [CASES[1], CASES[2], CASES[4]], ids=["dense", "dense-tail", "packed"])
def test_qk_normalisation_fused_into_the_core(case):
    """chunk_kda(..., normalize_qk=True) on unnormalised q and k: the forward results and every
    gradient that does not pass through the normalisation are bitwise those of
    chunk_kda(l2norm(q), l2norm(k), ...); dq and dk, which the fused backward derives from the
    unrounded core gradients, agree closely; and everything matches the oracle composition
    (reference stages: fwd/triton/l2norm_fwd.py:22, bwd/triton/l2norm_bwd.py:37)."""
    inp = _case(**case)
    gen = torch.Generator().manual_seed(96)
    scale_q = 0.5 + 3.0 * torch.rand(inp["q"].shape[:3], generator=gen)
    scale_k = 0.5 + 3.0 * torch.rand(inp["k"].shape[:3], generator=gen)
    raw_q = (inp["q"].float() * scale_q[..., None]).bfloat16()
    raw_k = (inp["k"].float() * scale_k[..., None]).bfloat16()
    do = torch.randn(inp["v"].shape, generator=gen).bfloat16()
    dst = 0.1 * torch.randn(inp["h0"].shape, generator=gen)
    cu = None if inp["cu_seqlens"] is None else inp["cu_seqlens"].cuda()
    if cu is not None:
        do[:, int(inp["cu_seqlens"][-1]):] = 0

    def run(fused):
        q, k, v = (t.cuda().requires_grad_() for t in (raw_q, raw_k, inp["v"]))
        g, beta, h0 = (inp[n].cuda().requires_grad_() for n in ("cum_gate", "beta", "h0"))
        if fused:
            o, st = kda_b200.chunk_kda(q, k, v, g, beta, h0, cu_seqlens=cu, output_final_state=True,
                                       normalize_qk=True)
        else:
            o, st = kda_b200.chunk_kda(kda_b200.l2norm(q), kda_b200.l2norm(k), v, g, beta, h0,
                                       cu_seqlens=cu, output_final_state=True)
        grads = torch.autograd.grad((o, st), (q, k, v, g, beta, h0), (do.cuda(), dst.cuda()))
        return dict(zip(("o", "state", "dq", "dk", "dv", "dg", "dbeta", "dh0"), (o, st) + grads))

    one, two = run(True), run(False)
    for name in ("o", "state", "dv", "dg", "dbeta", "dh0"):
        assert torch.equal(_active(inp, one[name]) if one[name].ndim > 3 and name not in ("state", "dh0")
                           else one[name],
                           _active(inp, two[name]) if two[name].ndim > 3 and name not in ("state", "dh0")
                           else two[name]), name
    assert torch.equal(_active(inp, one["dbeta"]), _active(inp, two["dbeta"]))
    for name in ("dq", "dk"):
        assert_normalised(_active(inp, one[name]).float(), _active(inp, two[name]).float(), 1e-2, name)
    # oracle: l2norm then the chunked recurrence, differentiated in fp32 on the CPU
    leaves = [t.float().requires_grad_() for t in (raw_q, raw_k, inp["v"])]
    leaves += [inp[n].clone().requires_grad_() for n in ("cum_gate", "beta", "h0")]
    qn = leaves[0] * torch.rsqrt((leaves[0] ** 2).sum(-1, keepdim=True) + 1e-6)
    kn = leaves[1] * torch.rsqrt((leaves[1] ** 2).sum(-1, keepdim=True) + 1e-6)
    ro, rs = orc.chunk_kda_ref(qn, kn, leaves[2], leaves[3], leaves[4], leaves[5], inp["cu_seqlens"])
    ref = torch.autograd.grad((ro, rs), leaves, (do.float(), dst))
    for name, r in zip(("dq", "dk", "dv", "dg", "dbeta", "dh0"), ref):
        a = one[name] if name == "dh0" else _active(inp, one[name])
        b = r if name == "dh0" else _active(inp, r)
        assert_normalised(a.float(), b, TOL, f"{name} vs oracle")
    assert_normalised(_active(inp, one["o"]).float(), _active(inp, ro.detach()), TOL, "output vs oracle")
    with pytest.raises(ValueError):
        kda_b200.chunk_kda(raw_q.cuda(), raw_k.cuda(), inp["v"].cuda(), inp["cum_gate"].cuda(),
                           inp["beta"].cuda(), cu_seqlens=cu, normalize_qk=True, recompute=True)


def test_dense_batch_equals_packed():
    """A dense batch and its explicit equal-length packing give bitwise-equal results
    (reference: test/test_kda_cute_forward.py:368-410)."""
    inp = _case(2, 192, 2, seed=7)
    res = _run_fused(inp)
    packed = dict(inp)
    for n in ("q", "k", "v", "cum_gate"):
        packed[n] = inp[n].reshape(1, 384, 2, 128)
    packed["beta"] = inp["beta"].reshape(1, 384, 2)
    packed["cu_seqlens"] = torch.tensor([0, 192, 384], dtype=torch.int32)
    res_p = _run_fused(packed)
    assert torch.equal(res["o"].reshape(1, 384, 2, 128), res_p["o"])
    assert torch.equal(res["state"], res_p["state"])


def test_causality_is_bitwise():
    """Perturbing tokens >= cut leaves outputs < cut bitwise unchanged
    (reference: test/test_kda_cute_forward.py:903-940)."""
    inp = _case(1, 256, 1, seed=8)
    base = _run_fused(inp)["o"]
    cut = 128
    pert = dict(inp)
    for n in ("q", "k", "v"):
        x = inp[n].clone()
        x[:, cut:] = x[:, cut:] * 1.5
        pert[n] = x
    other = _run_fused(pert)["o"]
    assert torch.equal(base[:, :cut], other[:, :cut])


def test_nan_poisoned_suffix_is_ignored():
    """Rows past cu_seqlens[-1] may hold anything (reference: test_kda_ragged_public_backward.py:125-139)."""
    inp = _case(1, 200, 1, seed=9, lengths=[70, 50])
    clean = _run_fused(inp)
    bad = dict(inp)
    for n in ("q", "k", "v", "cum_gate", "beta"):
        x = inp[n].clone()
        x[:, 120:] = float("nan")
        bad[n] = x
    res = _run_fused(bad)
    assert torch.equal(clean["o"][:, :120], res["o"][:, :120])
    assert torch.equal(clean["state"], res["state"])


def test_nan_poisoned_suffix_is_ignored_in_backward():
    """The same for the backward pass: NaN in every input row and in the output cotangent past
    cu_seqlens[-1] changes no gradient of the active prefix and no state gradient, bit for bit
    (reference: test/test_kda_ragged_bwd_wy.py:168-186, test_kda_ragged_public_backward.py:125-139).
    Both the kept-intermediates and the recompute backward are checked."""
    inp = _case(1, 200, 2, seed=10, lengths=[70, 0, 50])
    gen = torch.Generator().manual_seed(3)
    do = torch.randn(inp["v"].shape, generator=gen).bfloat16().float()
    dst = 0.1 * torch.randn(3, 2, 128, 128, generator=gen)
    bad = dict(inp)
    for n in ("q", "k", "v", "cum_gate", "beta"):
        x = inp[n].clone()
        x[:, 120:] = float("nan")
        bad[n] = x
    do_bad = do.clone()
    do_bad[:, 120:] = float("nan")
    for recompute in (False, True):
        clean = _run_fused(inp, do, dst, grad=True, recompute=recompute)
        res = _run_fused(bad, do_bad, dst, grad=True, recompute=recompute)
        for name in ("o", "dq", "dk", "dv", "dg", "dbeta"):
            assert torch.isfinite(res[name][:, :120].float()).all(), name
            assert torch.equal(clean[name][:, :120], res[name][:, :120]), name
        assert torch.equal(clean["state"], res["state"])
        assert torch.equal(clean["dh0"], res["dh0"])


def test_rejections():
    inp = _case(1, 64, 1, seed=1)
    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    with pytest.raises(ValueError):  # K != 128 on the fused bf16 path
        kda_b200.chunk_kda(c["q"][..., :64], c["k"][..., :64], c["v"], c["cum_gate"][..., :64],
                           c["beta"])
    with pytest.raises(ValueError):
        kda_b200.chunk_kda(c["q"], c["k"], c["v"], c["cum_gate"], c["beta"], impl="bogus")
    with pytest.raises(ValueError):
        kda_b200.chunk_kda(c["q"], c["k"], c["v"], c["cum_gate"], c["beta"], fastmath=True,
                           impl="reference")
    with pytest.raises(ValueError):  # packed input needs batch one
        kda_b200.chunk_kda(c["q"].repeat(2, 1, 1, 1), c["k"].repeat(2, 1, 1, 1),
                           c["v"].repeat(2, 1, 1, 1), c["cum_gate"].repeat(2, 1, 1, 1),
                           c["beta"].repeat(2, 1, 1),
                           cu_seqlens=torch.tensor([0, 64], dtype=torch.int32, device="cuda"))


def test_many_short_sequences():
    """300 packed sequences of 1..80 tokens (some empty): more offsets than the kernels keep in
    shared memory, so the work-item search reads them from global memory."""
    gen = torch.Generator().manual_seed(11)
    lengths = torch.randint(0, 81, (300,), generator=gen).tolist()
    lengths[7] = 0
    inp = _case(1, sum(lengths), 1, seed=12, lengths=lengths)
    got = _run_fused(inp)
    ref_o, ref_s = orc.chunk_kda_ref(inp["q"].float(), inp["k"].float(), inp["v"].float(), inp["cum_gate"],
                                     inp["beta"], inp["h0"], cu_seqlens=inp["cu_seqlens"])
    assert_normalised(_active(inp, got["o"]).float(), _active(inp, ref_o), TOL, "output")
    assert_normalised(got["state"], ref_s, TOL, "final states")


@pytest.mark.parametrize("normalize", [False, True], ids=["plain", "qk-norm"])
def test_repeated_runs_of_a_ragged_batch_give_the_same_bits(normalize):
    """Full chunks, partial tail chunks and empty sequences mixed, with enough (chunk, head) items
    for every persistent CTA to walk dozens of them: the two persistent kernels hand shared-memory
    tiles from one item to the next without a CTA barrier between full chunks, so a missing ordering
    would show up as run-to-run differences.  Twenty runs must agree bit for bit (outputs, final
    states and all gradients), and the device error word must stay clear."""
    from kda_b200 import _cabi

    gen = torch.Generator().manual_seed(21)
    picks = [1, 63, 64, 65, 127, 128, 200, 1000, 2048, 77, 0]
    lengths = [picks[i] for i in torch.randint(0, len(picks), (24,), generator=gen).tolist()]
    inp = orc.make_inputs(1, sum(lengths), 16, 128, 128, seed=22, lengths=lengths)
    q, k, v = (inp[n].bfloat16().cuda() for n in ("q", "k", "v"))
    gate, beta, cu = inp["cum_gate"].cuda(), inp["beta"].cuda(), inp["cu_seqlens"].cuda()
    do = torch.randn(v.shape, generator=torch.Generator(device="cuda").manual_seed(3), device="cuda").bfloat16()

    def run():
        ins = [t.detach().clone().requires_grad_(True) for t in (q, k, v, gate, beta)]
        o, st = kda_b200.chunk_kda(*ins, cu_seqlens=cu, output_final_state=True, normalize_qk=normalize)
        return (o, st) + torch.autograd.grad(o, ins, do)

    first = run()
    assert all(torch.isfinite(t.float()).all() for t in first)
    for _ in range(20):
        for name, a, b in zip(("o", "state", "dq", "dk", "dv", "dg", "dbeta"), first, run()):
            assert torch.equal(a, b), name
    torch.cuda.synchronize()
    assert _cabi.lib().kda_device_error_word() == 0


def test_library_calls_show_up_as_named_ranges_in_a_profiler_trace():
    """Under a torch profiler every C-ABI call of a forward + backward step is a named range
    (reference: profiler_range around each stage, fwd/cute/chunk_kda_fwd.py:94-119); without a
    profiler nothing is recorded (and nothing is paid)."""
    inp = _case(2, 256, 2, seed=2)
    do = torch.randn(inp["v"].shape, generator=torch.Generator().manual_seed(1))
    _run_fused(inp, do, grad=True)
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU,
                                            torch.profiler.ProfilerActivity.CUDA]) as prof:
        _run_fused(inp, do, grad=True)
        torch.cuda.synchronize()
    names = {e.name for e in prof.events()}
    assert any(n.startswith("kda_b200/kda_chunk_fwd") for n in names), sorted(names)[:40]
    assert "kda_b200/kda_chunk_bwd_saved" in names
    kernels = " ".join(sorted(names))
    assert "kda_prepare_tc_kernel" in kernels and "kda_bwd_chunk_tc_kernel" in kernels


def test_offsets_that_leave_the_buffer_are_skipped_and_reported():
    """cu_seqlens whose last sequence ends beyond the packed buffer (a value the host-side validation
    cannot see without a device synchronisation): every kernel of the chunked pair treats the chunks
    that do not lie inside the buffer as absent and raises its part of the device error word, the
    tensors stay finite, and the next, well-formed call is unaffected (reference: the device-side
    offset assertion of its scheduler, kda/chunk_scheduler.py:278-293)."""
    from kda_b200 import _cabi, ops

    inp = _case(1, 256, 2, seed=41)
    q, k, v = (inp[n].cuda() for n in ("q", "k", "v"))
    gate, beta = inp["cum_gate"].cuda(), inp["beta"].cuda()
    h0 = torch.zeros(2, 2, 128, 128, device="cuda")
    cu = torch.tensor([0, 100, 320], dtype=torch.int32, device="cuda")      # the buffer holds 256 tokens
    co = torch.tensor([0, 2, 6], dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    assert _cabi.lib().kda_device_error_word() == 0
    out, state, aqk, akk, saved = ops.chunk_fwd_saved_op(q, k, v, gate, beta, h0, cu, co, True)
    torch.cuda.synchronize()
    word = _cabi.lib().kda_device_error_word()
    assert word & 0xff == 9 and (word >> 16) & 0xff == 9, hex(word)      # state walk, prepare kernel
    assert torch.isfinite(out.float()).all() and torch.isfinite(state).all()
    do = torch.ones_like(out)
    grads = ops.chunk_bwd_saved_op(q, k, v, gate, beta, aqk, akk, saved, cu, co, do, None, h0, True)
    torch.cuda.synchronize()
    word = _cabi.lib().kda_device_error_word()
    assert word & 0xff == 9 and (word >> 8) & 0xff == 9, hex(word)       # state-gradient walk, chunk backward
    assert all(torch.isfinite(g.float()).all() for g in grads)
    # a well-formed call afterwards: clean error word, results as ever
    good = _case(1, 300, 2, seed=5, lengths=[65, 63, 0, 30, 128])
    got = _run_fused(good)
    torch.cuda.synchronize()
    assert _cabi.lib().kda_device_error_word() == 0
    ref_o, _ = orc.chunk_kda_ref(good["q"].float(), good["k"].float(), good["v"].float(), good["cum_gate"],
                                 good["beta"], good["h0"], cu_seqlens=good["cu_seqlens"])
    assert_normalised(_active(good, got["o"]).float(), _active(good, ref_o), TOL, "output after the reported call")


def test_a_bounded_wait_that_runs_out_reports_and_returns():
    """Every barrier wait of the tensor-memory kernels is bounded.  The library's self-test makes one
    run out on purpose (a barrier nothing arrives on, a few thousand polls): the kernel returns, the
    error word carries the code, it is cleared by reading, and the next normal call works."""
    from kda_b200 import _cabi

    lib = _cabi.lib()
    assert lib.kda_device_error_word() == 0
    assert lib.kda_selftest_bounded_wait(4096, _cabi.stream()) == 0
    torch.cuda.synchronize()
    assert lib.kda_device_error_word() == 2
    assert lib.kda_device_error_word() == 0
    inp = _case(1, 130, 1, seed=14)
    res = _run_fused(inp)
    ref_o, _ = orc.chunk_kda_ref(inp["q"].float(), inp["k"].float(), inp["v"].float(), inp["cum_gate"],
                                 inp["beta"], inp["h0"])
    assert_normalised(res["o"].float(), ref_o, TOL, "output after the self-test")
    assert lib.kda_device_error_word() == 0
    assert lib.kda_selftest_bounded_wait(0, _cabi.stream()) == -1
