"""Gate cumsum, l2norm, short convolution and chunk-offset parity through the C ABI."""

import pytest
import torch
import torch.nn.functional as F

import kda_b200
from kda_b200.chunk_schedule import chunk_capacity, prepare_ragged_chunk_metadata
from helpers import assert_normalised
from oracle import kda_oracle as orc

pytestmark = pytest.mark.gpu


def test_gate_golden(golden):
    g = {k: v.cuda() for k, v in golden("gate").items()}
    raw = g["raw"].bfloat16().requires_grad_(True)
    A_log = g["A_log"].clone().requires_grad_(True)
    bias = g["dt_bias"].clone().requires_grad_(True)
    out = kda_b200.bounded_gate_cumsum(raw, A_log, bias)
    torch.testing.assert_close(out, g["fwd"], atol=2e-5, rtol=1e-5)
    out.backward(g["dcum"])
    torch.testing.assert_close(raw.grad.float(), g["d_raw"], atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(A_log.grad, g["dA_log"], atol=5e-2, rtol=2e-2)
    torch.testing.assert_close(bias.grad, g["d_dt_bias"], atol=2e-2, rtol=2e-2)
    packed = kda_b200.bounded_gate_cumsum(g["raw"][:1, :131].bfloat16().contiguous(), g["A_log"],
                                          g["dt_bias"], cu_seqlens=g["cu_seqlens"])
    torch.testing.assert_close(packed, g["fwd_packed"], atol=2e-5, rtol=1e-5)


@pytest.mark.parametrize("chunk", [1, 16, 64])
def test_gate_chunk_sizes_and_packed_backward(chunk):
    gen = torch.Generator().manual_seed(3)
    raw = torch.randn(1, 300, 2, 64, generator=gen).bfloat16()
    A_log = 0.2 * torch.randn(2, generator=gen)
    bias = 0.3 * torch.randn(2, 64, generator=gen)
    dcum = torch.randn(1, 300, 2, 64, generator=gen)
    cu = torch.tensor([0, 65, 65, 128, 277], dtype=torch.int32)
    ref = orc.bounded_gate_cumsum_ref(raw, A_log, bias, chunk, -5.0, cu)
    r_raw, r_A, r_b = orc.bounded_gate_cumsum_bwd_ref(raw, A_log, bias, dcum, chunk, -5.0, cu)
    raw_g = raw.cuda().requires_grad_(True)
    A_g, b_g = A_log.cuda().requires_grad_(True), bias.cuda().requires_grad_(True)
    out = kda_b200.bounded_gate_cumsum(raw_g, A_g, b_g, chunk_size=chunk, cu_seqlens=cu.cuda())
    torch.testing.assert_close(out[:, :277].cpu(), ref[:, :277], atol=3e-5, rtol=1e-5)
    out.backward(dcum.cuda())
    torch.testing.assert_close(raw_g.grad[:, :277].float().cpu(), r_raw[:, :277], atol=2e-2,
                               rtol=2e-2)
    torch.testing.assert_close(A_g.grad.cpu(), r_A, atol=5e-2, rtol=2e-2)
    torch.testing.assert_close(b_g.grad.cpu(), r_b, atol=2e-2, rtol=2e-2)


def test_gate_offsets_that_leave_the_buffer_are_skipped_and_reported():
    """A last sequence that ends beyond the buffer: the gate kernels skip it and raise byte 3 of the
    device error word; the sequences inside the buffer are computed as ever."""
    from kda_b200 import _cabi

    gen = torch.Generator().manual_seed(4)
    raw = torch.randn(1, 300, 2, 64, generator=gen).bfloat16()
    A_log = 0.2 * torch.randn(2, generator=gen)
    bias = 0.3 * torch.randn(2, 64, generator=gen)
    good = torch.tensor([0, 65, 128], dtype=torch.int32)
    bad = torch.tensor([0, 65, 128, 400], dtype=torch.int32)          # the buffer holds 300 tokens
    ref = orc.bounded_gate_cumsum_ref(raw, A_log, bias, 64, -5.0, good)
    torch.cuda.synchronize()
    assert _cabi.lib().kda_device_error_word() == 0
    out = kda_b200.bounded_gate_cumsum(raw.cuda(), A_log.cuda(), bias.cuda(), chunk_size=64,
                                       cu_seqlens=bad.cuda())
    torch.cuda.synchronize()
    assert (_cabi.lib().kda_device_error_word() >> 24) & 0xff == 9
    assert torch.isfinite(out).all()
    torch.testing.assert_close(out[:, :128].cpu(), ref[:, :128], atol=3e-5, rtol=1e-5)
    out = kda_b200.bounded_gate_cumsum(raw.cuda(), A_log.cuda(), bias.cuda(), chunk_size=64,
                                       cu_seqlens=good.cuda())
    torch.cuda.synchronize()
    assert _cabi.lib().kda_device_error_word() == 0
    torch.testing.assert_close(out[:, :128].cpu(), ref[:, :128], atol=3e-5, rtol=1e-5)


def test_chunk_offsets_match_cpu():
    gen = torch.Generator().manual_seed(1)
    lens = torch.randint(0, 300, (5000,), generator=gen)
    lens[::7] = 0
    cu = torch.cat((torch.zeros(1, dtype=torch.long), lens.cumsum(0))).to(torch.int32)
    meta = prepare_ragged_chunk_metadata(cu.cuda(), int(cu[-1]) + 10, 64)
    want = torch.cat((torch.zeros(1, dtype=torch.long), ((lens + 63) // 64).cumsum(0)))
    assert torch.equal(meta.chunk_offsets.cpu().long(), want)
    assert meta.capacity == chunk_capacity(int(cu[-1]) + 10, 5000, 64) >= int(want[-1])


def test_l2norm_golden(golden):
    g = {k: v.cuda() for k, v in golden("l2norm").items()}
    x = g["x"].clone().requires_grad_(True)
    y = kda_b200.l2norm(x)
    torch.testing.assert_close(y, g["y"], atol=1e-6, rtol=1e-5)
    y.backward(g["dy"])
    torch.testing.assert_close(x.grad, g["dx"], atol=1e-5, rtol=1e-4)
    xb = g["x"].bfloat16()
    torch.testing.assert_close(kda_b200.l2norm(xb).float(), orc.l2norm_ref(xb.cpu())[0].float().cuda(),
                               atol=1e-2, rtol=1e-2)


def test_conv_golden(golden):
    g = {k: v.cuda() for k, v in golden("conv").items()}
    x = g["x"].clone().requires_grad_(True)
    w = g["w"].clone().requires_grad_(True)
    hist = g["hist"].clone().requires_grad_(True)
    y, final = kda_b200.causal_conv1d(x, w, activation="silu", initial_state=hist,
                                      return_final_state=True)
    torch.testing.assert_close(y, g["y"], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(final, g["final"], atol=0, rtol=0)
    dx, dw, dh = torch.autograd.grad(y, (x, w, hist), g["dy"])
    torch.testing.assert_close(dx, g["dx"], atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(dw, g["dw"], atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(dh, g["dhist"], atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("width", [1, 4, 5])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_conv_matches_pytorch(width, dtype):
    torch.manual_seed(0)
    x = torch.randn(2, 70, 32, device="cuda", dtype=dtype, requires_grad=True)
    w = torch.randn(32, width, device="cuda", dtype=dtype, requires_grad=True)
    dy = torch.randn_like(x)
    y = kda_b200.causal_conv1d(x, w, activation="silu")
    ref = F.silu(F.conv1d(F.pad(x.float().transpose(1, 2), (width - 1, 0)), w.float()[:, None],
                          groups=32).transpose(1, 2))
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    torch.testing.assert_close(y.float(), ref, atol=tol, rtol=tol)
    got = torch.autograd.grad(y, (x, w), dy)
    want = torch.autograd.grad(ref, (x, w), dy.float())
    torch.testing.assert_close(got[0].float(), want[0].float(), atol=3e-2 if dtype == torch.bfloat16 else 1e-4, rtol=3e-2)
    torch.testing.assert_close(got[1].float(), want[1].float(), atol=2e-1 if dtype == torch.bfloat16 else 1e-3, rtol=3e-2)


def test_conv_packed_and_decode():
    gen = torch.Generator().manual_seed(2)
    x = torch.randn(1, 90, 16, generator=gen)
    w = torch.randn(16, 4, generator=gen)
    hist = torch.randn(4, 3, 16, generator=gen)
    cu = torch.tensor([0, 2, 2, 40, 77], dtype=torch.int32)
    ref, ref_final = orc.causal_conv1d_ref(x, w, "silu", cu, hist)
    y, final = kda_b200.causal_conv1d(x.cuda(), w.cuda(), activation="silu", cu_seqlens=cu.cuda(),
                                      initial_state=hist.cuda(), return_final_state=True)
    torch.testing.assert_close(y[:, :77].cpu(), ref[:, :77], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(final.cpu(), ref_final, atol=0, rtol=0)
    # decode: continue each sequence by one token from its final history
    pool = torch.zeros(6, 3, 16)
    idx = torch.tensor([2, 0, 5, 1], dtype=torch.int32)
    for s, slot in enumerate(idx.tolist()):
        if slot > 0:
            pool[slot] = ref_final[s]
    xn = torch.randn(4, 16, generator=gen)
    pool_gpu = pool.cuda()
    yd = kda_b200.causal_conv1d_decode(xn.cuda(), w.cuda(), pool_gpu, activation="silu",
                                       state_indices=idx.cuda())
    for s, slot in enumerate(idx.tolist()):
        if slot <= 0:
            assert yd[s].abs().max() == 0
            continue
        ext = torch.cat((pool[slot], xn[s:s + 1]), 0)
        want = F.silu((ext * w.t()).sum(0))
        torch.testing.assert_close(yd[s].cpu(), want, atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(pool_gpu[slot].cpu(), ext[1:], atol=0, rtol=0)
    assert torch.equal(pool_gpu[[0, 3, 4]].cpu(), pool[[0, 3, 4]])


@pytest.mark.parametrize("offsets,capacity", [([0, 70, 150, 150], 192), ([0, 70, 150], 150),
                                              ([0, 5, 64, 64, 130, 321], 400), ([0, 128], 130)])
def test_conv_packed_backward_in_a_fixed_capacity_buffer(offsets, capacity):
    """bf16, width 4: input and weight gradients of packed sequences whose last 64-token run reaches
    into the unused tail of the buffer (the one-pass kernel leaves such a run to the edge kernels),
    against autograd through the CPU oracle; the tail of dx stays zero."""
    gen = torch.Generator().manual_seed(4)
    channels, active = 64, offsets[-1]
    x = torch.randn(1, capacity, channels, generator=gen).bfloat16()
    w = (0.5 * torch.randn(channels, 4, generator=gen)).bfloat16()
    dy = torch.randn(1, capacity, channels, generator=gen).bfloat16()
    dy[:, active:] = 0
    cu = torch.tensor(offsets, dtype=torch.int32)
    xr, wr = x.float().requires_grad_(), w.float().requires_grad_()
    ref, _ = orc.causal_conv1d_ref(xr, wr, "silu", cu, None)
    want = torch.autograd.grad(ref, (xr, wr), dy.float())
    xg, wg = x.cuda().requires_grad_(), w.cuda().requires_grad_()
    y = kda_b200.causal_conv1d(xg, wg, activation="silu", cu_seqlens=cu.cuda())
    torch.testing.assert_close(y[:, :active].float().cpu(), ref[:, :active].detach(), atol=2e-2, rtol=2e-2)
    got = torch.autograd.grad(y, (xg, wg), dy.cuda())
    torch.testing.assert_close(got[0][:, :active].float().cpu(), want[0][:, :active], atol=3e-2, rtol=3e-2)
    assert got[0][:, active:].abs().max() == 0 if active < capacity else True
    torch.testing.assert_close(got[1].float().cpu(), want[1], atol=2e-1, rtol=3e-2)


@pytest.mark.parametrize("dtype,dim,rows,tol", [
    (torch.bfloat16, 128, (3, 37, 4), 2e-2), (torch.float16, 64, (1, 130, 2), 4e-3),
    (torch.bfloat16, 256, (2, 19, 1), 2e-2), (torch.float32, 128, (2, 33, 4), 2e-5),
    (torch.float32, 96, (1, 21, 3), 2e-5), (torch.bfloat16, 128, (1, 4099, 8), 2e-2),
])
def test_gated_output_norm(dtype, dim, rows, tol):
    """RMSNorm * weight * sigmoid(gate) epilogue, values and the three gradients, against the fp32
    oracle evaluated on the same (rounded) inputs."""
    gen = torch.Generator().manual_seed(dim + rows[1])
    o = torch.randn(*rows, dim, generator=gen).to(dtype)
    z = (2 * torch.randn(*rows, dim, generator=gen)).to(dtype)
    w = 1 + 0.2 * torch.randn(dim, generator=gen)
    dy = torch.randn(*rows, dim, generator=gen).to(dtype)
    ro, rz, rw = (t.float().clone().requires_grad_() for t in (o, z, w))
    ref = orc.gated_output_norm_ref(ro, rz, rw, 1e-5)
    rgo, rgz, rgw = torch.autograd.grad(ref, (ro, rz, rw), dy.float())
    go, gz, gw = (t.detach().cuda().requires_grad_() for t in (o, z, w))
    y = kda_b200.gated_output_norm(go, gz, gw, 1e-5)
    assert y.dtype == dtype
    y.backward(dy.cuda())
    assert_normalised(y.float(), ref.detach(), tol, "epilogue output")
    assert_normalised(go.grad.float(), rgo, tol, "epilogue d_o")
    assert_normalised(gz.grad.float(), rgz, tol, "epilogue d_gate_logits")
    assert_normalised(gw.grad.float(), rgw, max(tol / 4, 2e-5), "epilogue d_weight")
