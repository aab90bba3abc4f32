"""Compiler contract of the torch.library operators: every operator of the ``kda_b200`` namespace
goes through ``torch.library.opcheck`` (schema: declared aliasing and mutation match what the CUDA
implementation does; fake tensor: the registered meta implementation returns the shapes, dtypes,
devices and strides of the real one), and the public chunked op runs forward and backward under
``torch.compile(fullgraph=True)``.  The reference checks its operators the same way
(test/test_kda_cute_forward.py:616-693, test/test_kda_ragged_autograd_ops.py:25-100,
test/test_kda_recurrent.py:378-411)."""

import pytest
import torch

import kda_b200
from kda_b200 import _cabi
from kda_b200.chunk_schedule import prepare_ragged_chunk_metadata
from oracle import kda_oracle as orc

pytestmark = pytest.mark.gpu
CHECKS = ("test_schema", "test_faketensor")
ops = torch.ops.kda_b200


def _chunk_inputs(batch, tokens, heads, lengths=None, seed=61):
    inp = orc.make_inputs(batch, tokens, heads, 128, 128, seed=seed, with_state=True, lengths=lengths)
    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    for n in ("q", "k", "v"):
        c[n] = c[n].bfloat16()
    return c


def _check(op, *args, **kwargs):
    torch.library.opcheck(op, args, kwargs, test_utils=CHECKS)


def test_chunk_forward_ops_dense():
    c = _chunk_inputs(2, 130, 2)
    args = (c["q"], c["k"], c["v"], c["cum_gate"], c["beta"])
    _check(ops.kda_chunk_fwd.default, *args, c["h0"], True)
    _check(ops.kda_chunk_fwd.default, *args, None, True)
    _check(ops.kda_chunk_fwd_with_state.default, *args, c["h0"], True)
    _check(ops.kda_chunk_fwd_saved.default, *args, c["h0"], None, None, True)
    _check(ops.kda_chunk_fwd_saved.default, *args, None, None, None, False)


def test_chunk_forward_ops_packed():
    c = _chunk_inputs(1, 300, 2, lengths=[65, 0, 100, 64])
    meta = prepare_ragged_chunk_metadata(c["cu_seqlens"], 300, 64)
    args = (c["q"], c["k"], c["v"], c["cum_gate"], c["beta"], c["h0"], meta.cu_seqlens,
            meta.chunk_offsets)
    _check(ops.kda_chunk_fwd_ragged.default, *args, True)
    _check(ops.kda_chunk_fwd_ragged_with_state.default, *args, True)
    _check(ops.kda_chunk_fwd_saved.default, *args, True)
    _check(ops.kda_prepare_chunk_offsets.default, c["cu_seqlens"], 300, 64)


@pytest.mark.parametrize("packed", [False, True], ids=["dense", "packed"])
def test_chunk_backward_ops(packed):
    if packed:
        c = _chunk_inputs(1, 300, 2, lengths=[65, 0, 100, 64])
        meta = prepare_ragged_chunk_metadata(c["cu_seqlens"], 300, 64)
        cu, co = meta.cu_seqlens, meta.chunk_offsets
    else:
        c = _chunk_inputs(2, 130, 2)
        cu = co = None
    args = (c["q"], c["k"], c["v"], c["cum_gate"], c["beta"])
    out, state, aqk, akk, saved = ops.kda_chunk_fwd_saved(*args, c["h0"], cu, co, True)
    gen = torch.Generator(device="cuda").manual_seed(1)
    do = torch.randn(out.shape, generator=gen, device="cuda").bfloat16()
    dst = torch.randn(state.shape, generator=gen, device="cuda")
    _check(ops.kda_chunk_bwd.default, *args, aqk, akk, cu, co, do, None, None, False, True)
    _check(ops.kda_chunk_bwd.default, *args, aqk, akk, cu, co, do, dst, c["h0"], False, True)
    _check(ops.kda_chunk_bwd_with_state_grad.default, *args, aqk, akk, cu, co, do, dst, c["h0"], False,
           True)
    _check(ops.kda_chunk_bwd_saved.default, *args, aqk, akk, saved, cu, co, do, dst, c["h0"], True)
    _check(ops.kda_chunk_bwd_saved.default, *args, aqk, akk, saved, cu, co, do, None, None, False)
    _check(ops.kda_chunk_bwd_state_saved.default, c["cum_gate"], aqk, saved, cu, co, do, dst)
    _check(ops.kda_chunk_bwd_state_saved.default, c["cum_gate"], aqk, saved, cu, co, do, None)


@pytest.mark.parametrize("packed", [False, True], ids=["dense", "packed"])
def test_chunk_ops_with_fused_qk_normalisation(packed):
    if packed:
        c = _chunk_inputs(1, 300, 2, lengths=[65, 0, 100, 64])
        meta = prepare_ragged_chunk_metadata(c["cu_seqlens"], 300, 64)
        cu, co = meta.cu_seqlens, meta.chunk_offsets
    else:
        c = _chunk_inputs(2, 130, 2)
        cu = co = None
    args = (3 * c["q"], 2 * c["k"], c["v"], c["cum_gate"], c["beta"])
    _check(ops.kda_chunk_fwd_qknorm.default, *args, c["h0"], cu, co, True, True, 1e-6)
    _check(ops.kda_chunk_fwd_qknorm.default, *args, None, cu, co, False, False, 1e-6)
    out, state, aqk, akk, saved, rq, rk = ops.kda_chunk_fwd_qknorm(*args, c["h0"], cu, co, True, True, 1e-6)
    gen = torch.Generator(device="cuda").manual_seed(1)
    do = torch.randn(out.shape, generator=gen, device="cuda").bfloat16()
    dst = torch.randn(state.shape, generator=gen, device="cuda")
    _check(ops.kda_chunk_bwd_qknorm.default, *args, aqk, akk, saved, rq, rk, cu, co, do, dst, c["h0"], True)
    _check(ops.kda_chunk_bwd_qknorm.default, *args, aqk, akk, saved, rq, rk, cu, co, do, None, None, False)


def test_saved_buffer_of_the_fake_matches_the_library():
    """The meta implementation of kda_chunk_fwd_saved sizes the kept-intermediates buffer with the
    library's own shape-only function, for dense and packed inputs."""
    lib = _cabi.lib()
    c = _chunk_inputs(2, 130, 2)
    real = ops.kda_chunk_fwd_saved(c["q"], c["k"], c["v"], c["cum_gate"], c["beta"], None, None, None,
                                   False)[4]
    assert real.numel() == lib.kda_chunk_fwd_dense_workspace_bytes(2, 130, 2, 1)
    assert real.numel() >= lib.kda_chunk_bwd_workspace_bytes(2 * 130, 2, 2 * 3)


def test_recurrent_ops():
    inp = orc.make_inputs(3, 5, 2, 128, 128, seed=62, with_state=True)
    c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    args = (c["q"].bfloat16(), c["k"].bfloat16(), c["v"].bfloat16(), c["gate_log2"], c["beta"])
    _check(ops.kda_recurrent_fwd.default, *args, c["h0"], None, True)
    _check(ops.kda_recurrent_fwd_no_state.default, *args, None, None, True)
    one = tuple(t[:, :1].contiguous() for t in args)
    pool = torch.cat((torch.zeros_like(c["h0"][:1]), c["h0"]), 0)
    idx = torch.tensor([2, 0, 3], dtype=torch.int32, device="cuda")
    _check(ops.kda_recurrent_fwd_paged.default, *one, pool, idx, None, True)


def test_gate_l2norm_and_epilogue_ops():
    gen = torch.Generator(device="cuda").manual_seed(63)
    raw = torch.randn(2, 100, 2, 128, generator=gen, device="cuda").bfloat16()
    a_log = 0.3 * torch.randn(2, generator=gen, device="cuda")
    dt_bias = 0.3 * torch.randn(2, 128, generator=gen, device="cuda")
    dcum = torch.randn(2, 100, 2, 128, generator=gen, device="cuda")
    _check(ops.kda_bounded_gate_fwd_dense.default, raw, a_log, dt_bias, 64, -5.0)
    _check(ops.kda_bounded_gate_bwd.default, raw, a_log, dt_bias, dcum, None, None, 64, -5.0)
    cu = torch.tensor([0, 70, 70, 180], dtype=torch.int32, device="cuda")
    meta = prepare_ragged_chunk_metadata(cu, 200, 64)
    raw1 = torch.randn(1, 200, 2, 128, generator=gen, device="cuda").bfloat16()
    dcum1 = torch.randn(1, 200, 2, 128, generator=gen, device="cuda")
    _check(ops.kda_bounded_gate_fwd_ragged.default, raw1, a_log, dt_bias, meta.cu_seqlens,
           meta.chunk_offsets, 64, -5.0)
    _check(ops.kda_bounded_gate_bwd.default, raw1, a_log, dt_bias, dcum1, meta.cu_seqlens,
           meta.chunk_offsets, 64, -5.0)
    x = torch.randn(2, 100, 2, 128, generator=gen, device="cuda").bfloat16()
    _check(ops.kda_l2norm_fwd.default, x, 1e-6)
    y, rstd = ops.kda_l2norm_fwd(x, 1e-6)
    _check(ops.kda_l2norm_bwd.default, y, rstd, torch.randn_like(y))
    weight = 1 + 0.1 * torch.randn(128, generator=gen, device="cuda")
    _check(ops.kda_output_gate_fwd.default, x, raw, weight, 1e-5)
    _check(ops.kda_output_gate_bwd.default, x, raw, weight, torch.randn_like(x), 1e-5)


def test_short_conv_and_decode_ops():
    gen = torch.Generator(device="cuda").manual_seed(64)
    channels, width = 3 * 2 * 128, 4
    x = torch.randn(2, 70, channels, generator=gen, device="cuda").bfloat16()
    w = (0.5 * torch.randn(channels, width, generator=gen, device="cuda")).bfloat16()
    state = torch.randn(2, width - 1, channels, generator=gen, device="cuda").bfloat16()
    dy = torch.randn_like(x)
    _check(ops.short_conv_fwd.default, x, w, None, state, activation="silu")
    _check(ops.short_conv_fwd.default, x, w)
    _check(ops.short_conv_bwd.default, x, w, dy, None, state, activation="silu", state_grad=True)
    _check(ops.short_conv_bwd.default, x, w, dy)
    cu = torch.tensor([0, 30, 30, 100], dtype=torch.int32, device="cuda")
    x1 = torch.randn(1, 120, channels, generator=gen, device="cuda").bfloat16()
    _check(ops.short_conv_fwd.default, x1, w, cu, None, activation="silu")
    _check(ops.short_conv_bwd.default, x1, w, torch.randn_like(x1), cu, None, activation="silu")
    tok = torch.randn(3, channels, generator=gen, device="cuda").bfloat16()
    pool = torch.randn(5, width - 1, channels, generator=gen, device="cuda").bfloat16()
    idx = torch.tensor([4, 0, 2], dtype=torch.int32, device="cuda")
    _check(ops.short_conv_decode.default, tok, w, pool, idx, activation="silu")
    raw = torch.randn(3, 2, 128, generator=gen, device="cuda").bfloat16()
    a_log = 0.3 * torch.randn(2, generator=gen, device="cuda")
    dt_bias = 0.3 * torch.randn(2, 128, generator=gen, device="cuda")
    _check(ops.kda_decode_prep.default, tok, w, pool, idx, raw, a_log, dt_bias, 2, "silu", -5.0, 1e-6)


def test_every_operator_of_the_namespace_is_covered():
    """A new operator must get an opcheck above: the list is compared with the registered schemas."""
    covered = {
        "kda_chunk_fwd", "kda_chunk_fwd_with_state", "kda_chunk_fwd_ragged",
        "kda_chunk_fwd_ragged_with_state", "kda_chunk_fwd_saved", "kda_chunk_bwd",
        "kda_chunk_bwd_with_state_grad", "kda_chunk_bwd_saved", "kda_chunk_bwd_state_saved",
        "kda_chunk_fwd_qknorm",
        "kda_chunk_bwd_qknorm", "kda_recurrent_fwd",
        "kda_recurrent_fwd_no_state", "kda_recurrent_fwd_paged", "kda_prepare_chunk_offsets",
        "kda_bounded_gate_fwd_dense", "kda_bounded_gate_fwd_ragged", "kda_bounded_gate_bwd",
        "kda_l2norm_fwd", "kda_l2norm_bwd", "kda_output_gate_fwd", "kda_output_gate_bwd",
        "short_conv_fwd", "short_conv_bwd", "short_conv_decode", "kda_decode_prep"}
    registered = {name.split("::")[1].split(".")[0]
                  for name in torch._C._dispatch_get_all_op_names() if name.startswith("kda_b200::")}
    assert registered == covered, registered ^ covered


@pytest.mark.parametrize("packed", [False, True], ids=["dense", "packed"])
def test_chunk_kda_under_torch_compile_fullgraph(packed):
    """Forward and backward of the public op traced as one graph (no graph breaks); results equal
    the eager call bit for bit, since the same kernels run."""
    if packed:
        c = _chunk_inputs(1, 300, 2, lengths=[65, 0, 100, 64], seed=65)
    else:
        c = _chunk_inputs(2, 192, 2, seed=65)
    cu = c["cu_seqlens"]

    def fn(q, k, v, g, beta, h0):
        return kda_b200.chunk_kda(q, k, v, g, beta, h0, cu_seqlens=cu, output_final_state=True)

    compiled = torch.compile(fn, fullgraph=True, backend="aot_eager")
    gen = torch.Generator(device="cuda").manual_seed(2)
    do = torch.randn(c["v"].shape, generator=gen, device="cuda").bfloat16()
    dst = torch.randn(c["h0"].shape, generator=gen, device="cuda")
    if packed:
        do[:, int(cu[-1]):] = 0
    results = []
    for f in (fn, compiled):
        leaves = [c[n].detach().clone().requires_grad_() for n in ("q", "k", "v", "cum_gate", "beta", "h0")]
        o, s = f(*leaves)
        grads = torch.autograd.grad((o, s), leaves, (do, dst))
        results.append((o, s) + grads)
    active = slice(None) if not packed else slice(0, int(cu[-1]))
    for name, a, b in zip(("o", "state", "dq", "dk", "dv", "dg", "dbeta", "dh0"), *results):
        if a.ndim == 4 and a.shape[1] == c["q"].shape[1]:
            a, b = a[:, active], b[:, active]
        elif a.ndim == 3 and name == "dbeta":
            a, b = a[:, active], b[:, active]
        assert torch.equal(a, b), name
