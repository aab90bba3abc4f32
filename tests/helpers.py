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


def assert_budget(actual, golden, low_precision, name, dtype=torch.bfloat16):
    """The reference's data-derived error budget (test/test_kda_kernels.py:141-156,
    attn_gym/testing/kda.py:48-64): the kernel may be off the fp64 result by at most twice what an
    independent low-precision evaluation of the same mathematics is off, plus a rounding band of
    two ulps of ``dtype`` at the largest magnitude."""
    g = golden.detach().double().cpu()
    band = torch.finfo(dtype).eps * float(g.abs().max())
    a_err = float((actual.detach().double().cpu() - g).abs().max())
    r_err = float((low_precision.detach().double().cpu() - g).abs().max())
    budget = 2.0 * r_err + 2.0 * band
    assert a_err <= budget, (f"{name}: kernel error {a_err:.3e} exceeds budget {budget:.3e} "
                             f"(low-precision reference error {r_err:.3e}, band {band:.3e})")
