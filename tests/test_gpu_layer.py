"""The caller module ``KDAAttention`` (conv -> l2norm -> gate -> chunk_kda -> output epilogue) on
the CUDA kernels: against its own eager fp32 backend, packed input against a per-sequence loop, and
fixed-capacity packed buffers with a poisoned suffix
(reference: test/test_kda_training_example.py:161-325)."""

import pytest
import torch

from kda_b200.layer import KDAAttention
from helpers import assert_normalised

pytestmark = pytest.mark.gpu


def _models(hidden, heads, seed, **kw):
    torch.manual_seed(seed)
    fused = KDAAttention(hidden, heads, 128, backend="fused", device="cuda", **kw)
    with torch.no_grad():
        fused.A_log.copy_(0.3 * torch.randn_like(fused.A_log))
        fused.dt_bias.copy_(0.3 * torch.randn_like(fused.dt_bias))
        fused.output_norm_weight.copy_(1 + 0.1 * torch.randn_like(fused.output_norm_weight))
    # the eager backend with the same bf16 projections, so the comparison isolates the kernels
    ref = KDAAttention(hidden, heads, 128, backend="reference", device="cuda",
                       compute_dtype=torch.bfloat16, **kw)
    ref.load_state_dict(fused.state_dict())
    return fused, ref


GATE_PATH = ("A_log", "dt_bias", "f_a_proj.weight", "f_b_proj.weight")


def test_fused_layer_matches_its_eager_backend(monkeypatch):
    import kda_b200.layer as layer_module

    fused, ref = _models(64, 2, seed=71)
    x = torch.randn(2, 130, 64, device="cuda")
    h0 = 0.1 * torch.randn(2, 2, 128, 128, device="cuda")
    c0 = torch.randn(2, 3, 3 * 2 * 128, device="cuda")
    cot = torch.randn(2, 130, 64, device="cuda")
    seen = {}
    gate_op = layer_module._bounded_gate_cumsum

    def record_gate(raw_gate, *args, **kwargs):
        out = gate_op(raw_gate, *args, **kwargs)
        out.retain_grad()
        seen["cumulative_gate"] = out
        return out

    monkeypatch.setattr(layer_module, "_bounded_gate_cumsum", record_gate)
    results = []
    for model in (fused, ref):
        xin = x.clone().requires_grad_()
        out = model(xin, h0, initial_conv_state=c0, return_final_state=True)
        params = list(model.parameters())
        grads = torch.autograd.grad(out.hidden_states, [xin] + params, cot)
        results.append((out, grads))
    (fo, fg), (ro, rg) = results
    assert fo.hidden_states.dtype == torch.float32
    assert_normalised(fo.hidden_states, ro.hidden_states, 3e-2, "layer output")
    assert_normalised(fo.final_state, ro.final_state, 3e-2, "final recurrent state")
    assert_normalised(fo.final_conv_state.float(), ro.final_conv_state.float(), 2e-2, "final conv state")
    names = ["hidden"] + [n for n, _ in fused.named_parameters()]
    got = dict(zip(names, fg))
    for name, a, b in zip(names, fg, rg):
        if name not in GATE_PATH:
            assert_normalised(a.float(), b.float(), 5e-2, f"gradient of {name}")
    # The gate parameters receive their gradient as a chunk-local reverse prefix sum of d(cumulative
    # gate) summed over all tokens: large terms of both signs that nearly cancel, so two bf16
    # evaluations of the core agree on d(cumulative gate) to 1e-2 and still differ visibly in these
    # sums.  Their wiring is checked exactly instead: the eager fp32 gate, differentiated with the
    # d(cumulative gate) the fused core produced, must give the fused layer's gradients.
    dg = seen["cumulative_gate"].grad
    hidden = x.to(torch.bfloat16)
    raw = fused._linear(fused._linear(hidden, fused.f_a_proj), fused.f_b_proj).view(2, 130, 2, 128)
    z = raw.float() + fused.dt_bias
    gate = fused.lower_bound * torch.sigmoid(fused.A_log.exp().view(1, 1, -1, 1) * z) * 1.4426950408889634
    pad = (-130) % 64
    cum = torch.nn.functional.pad(gate, (0, 0, 0, 0, 0, pad)).view(2, -1, 64, 2, 128).cumsum(2)
    cum = cum.view(2, -1, 2, 128)[:, :130]
    wrt = [fused.A_log, fused.dt_bias, fused.f_a_proj.weight, fused.f_b_proj.weight]
    want = torch.autograd.grad(cum, wrt, dg)
    for name, b in zip(GATE_PATH, want):
        assert_normalised(got[name].float(), b.float(), 3e-2, f"gradient of {name} (same d gate)")


def test_packed_input_matches_a_loop_over_the_sequences():
    fused, _ = _models(32, 1, seed=72)
    offsets = (0, 65, 65, 128, 200)
    packed = torch.randn(1, offsets[-1], 32, device="cuda", requires_grad=True)
    loop = packed.detach().clone().requires_grad_()
    cu = torch.tensor(offsets, device="cuda", dtype=torch.int32)
    h0 = 0.1 * torch.randn(4, 1, 128, 128, device="cuda")
    got = fused(packed, h0, cu_seqlens=cu, return_final_state=True)
    parts, states, conv_states = [], [], []
    for i, (a, b) in enumerate(zip(offsets[:-1], offsets[1:])):
        if a == b:
            states.append(h0[i:i + 1])
            conv_states.append(torch.zeros(1, 3, 3 * 128, device="cuda", dtype=torch.bfloat16))
            continue
        one = fused(loop[:, a:b], h0[i:i + 1], return_final_state=True)
        parts.append(one.hidden_states)
        states.append(one.final_state)
        conv_states.append(one.final_conv_state)
    want = torch.cat(parts, 1)
    torch.testing.assert_close(got.hidden_states, want)
    assert torch.equal(got.final_state, torch.cat(states, 0))
    assert torch.equal(got.final_conv_state, torch.cat(conv_states, 0))
    cot = torch.randn_like(want)
    g1 = torch.autograd.grad(got.hidden_states, packed, cot)[0]
    g2 = torch.autograd.grad(want, loop, cot)[0]
    torch.testing.assert_close(g1, g2, rtol=3e-2, atol=3e-2)


def test_fixed_capacity_buffer_with_poisoned_suffix():
    """A packed buffer longer than cu_seqlens[-1], NaN past the end, mask_inactive_capacity=True:
    outputs and every gradient equal those of the exactly sized run."""
    fused, _ = _models(32, 1, seed=73, mask_inactive_capacity=True)
    params = list(fused.parameters())
    capacity, active = 192, 150
    x = torch.randn(1, capacity, 32, device="cuda")
    cot = torch.randn(1, capacity, 32, device="cuda")
    cu = torch.tensor([0, 70, 150, 150], device="cuda", dtype=torch.int32)
    exact_x = x[:, :active].clone().requires_grad_()
    exact = fused(exact_x, cu_seqlens=torch.tensor([0, 70, 150], device="cuda", dtype=torch.int32))
    exact_g = torch.autograd.grad(exact.hidden_states, [exact_x] + params, cot[:, :active])
    bad_x, bad_cot = x.clone(), cot.clone()
    bad_x[:, active:] = float("nan")
    bad_cot[:, active:] = float("nan")
    bad_x.requires_grad_()
    got = fused(bad_x, cu_seqlens=cu)
    got_g = torch.autograd.grad(got.hidden_states, [bad_x] + params, bad_cot)
    torch.testing.assert_close(got.hidden_states[:, :active], exact.hidden_states)
    torch.testing.assert_close(got_g[0][:, :active], exact_g[0], rtol=3e-2, atol=3e-2)
    for (name, _), a, b in zip(fused.named_parameters(), got_g[1:], exact_g[1:]):
        assert torch.isfinite(a).all(), name
        assert_normalised(a.float(), b.float(), 3e-2, f"gradient of {name}")


def test_fused_qk_norm_equals_the_separate_l2norm_launches():
    """The layer with the normalisation inside the core against the same layer running l2norm as
    separate launches: same forward bits, gradients of the hidden states close."""
    fused, _ = _models(64, 2, seed=74)
    apart = KDAAttention(64, 2, 128, backend="fused", device="cuda", fuse_qk_norm=False)
    apart.load_state_dict(fused.state_dict())
    x = torch.randn(2, 200, 64, device="cuda")
    cot = torch.randn(2, 200, 64, device="cuda")
    res = []
    for model in (fused, apart):
        xin = x.clone().requires_grad_()
        out = model(xin, return_final_state=True)
        res.append((out, torch.autograd.grad(out.hidden_states, xin, cot)[0]))
    assert torch.equal(res[0][0].hidden_states, res[1][0].hidden_states)
    assert torch.equal(res[0][0].final_state, res[1][0].final_state)
    assert_normalised(res[0][1], res[1][1], 2e-2, "hidden gradient")


def test_constructor_and_forward_checks():
    with pytest.raises(ValueError):
        KDAAttention(32, 1, 64, backend="fused")
    with pytest.raises(ValueError):
        KDAAttention(32, 1, 128, backend="cuda")
    model = KDAAttention(32, 1, 128, backend="reference", device="cuda")
    with pytest.raises(ValueError):
        model(torch.randn(1, 8, 32, device="cuda"),
              cu_seqlens=torch.tensor([0, 8], device="cuda", dtype=torch.int32))
    with pytest.raises(ValueError):
        model(torch.randn(1, 8, 16, device="cuda"))
