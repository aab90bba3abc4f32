"""Shared helpers of the GPU parity tests."""

import torch


def norm_err(actual, ref):
    """max |actual - ref| divided by max |ref| (errors are judged on normalised tensors)."""
    if actual.is_cuda and ref.is_cuda and actual.numel() > (1 << 24):
        # large tensors stay on the GPU (fp32 is ample for a max-norm of bf16-sized errors)
        a, r = actual.detach().float(), ref.detach().float()
        return float((a - r).abs().max() / max(float(r.abs().max()), 1e-12))
    a, r = actual.detach().double().cpu(), ref.detach().double().cpu()
    return float((a - r).abs().max() / max(float(r.abs().max()), 1e-12))


def assert_normalised(actual, ref, tol, name):
    assert torch.isfinite(actual).all(), f"{name}: non-finite values"
    err = norm_err(actual, ref)
    assert err <= tol, f"{name}: normalised max error {err:.3e} > {tol:.1e}"


def to_cuda(inp, dtype=None):
    out = {}
    for key, val in inp.items():
        if torch.is_tensor(val):
            val = val.cuda()
            if dtype is not None and key in ("q", "k", "v"):
                val = val.to(dtype)
        out[key] = val
    return out


def bf16_round(inp):
    """The inputs the bf16 kernels actually see: q, k, v rounded to bf16, kept as fp32 values."""
    out = dict(inp)
    for key in ("q", "k", "v"):
        out[key] = inp[key].bfloat16().float()
    return out
