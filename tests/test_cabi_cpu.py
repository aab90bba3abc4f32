"""CPU-side checks: the shared library builds, loads and exports every symbol the header declares;
host-side logic (validation, chunk capacity, reference impl, masks) behaves like the reference."""

import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    import __graft_entry__  # noqa: F401  (path setup)
    from kda_b200 import _cabi, build

    build.build()
    header = open(os.path.join(ROOT, "include", "kda_b200.h")).read()
    declared = set(re.findall(r"^(?:int|int64_t|const char\*)\s+(kda_[a-z0-9_]+)\s*\(", header, re.M))
    lib = _cabi.lib()
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/kda_b200.h but not exported"
    assert declared == set(_cabi.exported_symbols())
    assert lib.kda_b200_version() >= 100
    assert lib.kda_chunk_fwd_workspace_bytes(64, 2) == 4 * 64 * 2 * 128 * 2


def test_fused_path_has_no_cpu_fallback():
    import kda_b200
    from oracle import kda_oracle as orc

    inp = orc.make_inputs(1, 64, 1, 128, 128, seed=1)
    with pytest.raises(ValueError):
        kda_b200.chunk_kda(inp["q"], inp["k"], inp["v"], inp["cum_gate"], inp["beta"])
    with pytest.raises(ValueError):
        kda_b200.recurrent_kda(inp["q"], inp["k"], inp["v"], inp["gate_log2"], inp["beta"])


def test_reference_impl_matches_oracle():
    import kda_b200
    from oracle import kda_oracle as orc

    inp = orc.make_inputs(1, 150, 2, 32, 48, seed=2, with_state=True, lengths=[70, 0, 61])
    o, s = kda_b200.chunk_kda(inp["q"], inp["k"], inp["v"], inp["cum_gate"], inp["beta"], inp["h0"],
                              cu_seqlens=inp["cu_seqlens"], output_final_state=True,
                              impl="reference")
    ro, rs = orc.chunk_kda_ref(inp["q"], inp["k"], inp["v"], inp["cum_gate"], inp["beta"],
                               inp["h0"], inp["cu_seqlens"])
    torch.testing.assert_close(o, ro, atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(s, rs, atol=1e-5, rtol=1e-4)
    o2, s2 = kda_b200.recurrent_kda(inp["q"], inp["k"], inp["v"], inp["gate_log2"], inp["beta"],
                                    inp["h0"], cu_seqlens=inp["cu_seqlens"],
                                    output_final_state=True, impl="reference")
    torch.testing.assert_close(o2, ro, atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(s2, rs, atol=1e-5, rtol=1e-4)
    assert torch.equal(s[1], inp["h0"][1])


def test_validation_errors():
    import kda_b200
    from oracle import kda_oracle as orc

    inp = orc.make_inputs(1, 8, 1, 16, 16, seed=1)
    q, k, v, g, b = inp["q"], inp["k"], inp["v"], inp["gate_log2"], inp["beta"]
    with pytest.raises(ValueError):
        kda_b200.recurrent_kda(q[0], k, v, g, b, impl="reference")
    with pytest.raises(ValueError):
        kda_b200.recurrent_kda(q, k[:, :4], v, g, b, impl="reference")
    with pytest.raises(ValueError):
        kda_b200.recurrent_kda(q, k, v, g, b[:, :4], impl="reference")
    with pytest.raises(TypeError):
        kda_b200.recurrent_kda(q.double(), k.double(), v.double(), g.double(), b.double(),
                               impl="reference")
    with pytest.raises(ValueError):  # cu_seqlens must be integer offsets on the same device
        kda_b200.recurrent_kda(q, k, v, g, b, cu_seqlens=torch.tensor([0.0, 8.0]), impl="reference")
    with pytest.raises(ValueError):
        kda_b200.recurrent_kda(q, k, v, g, b, torch.zeros(2, 1, 16, 16), impl="reference")
    with pytest.raises(ValueError):
        kda_b200.recurrent_kda(q, k, v, g, b, torch.zeros(3, 1, 16, 16),
                               state_indices=torch.zeros(1, dtype=torch.int32), impl="reference")


def test_chunk_capacity_bound():
    from kda_b200.chunk_schedule import chunk_capacity

    assert chunk_capacity(0, 3, 64) == 0
    assert chunk_capacity(5, 8, 64) == 5
    assert chunk_capacity(200, 3, 64) == 3 + 197 // 64
    gen = torch.Generator().manual_seed(0)
    for _ in range(50):
        n = int(torch.randint(1, 9, (1,), generator=gen))
        lens = torch.randint(0, 200, (n,), generator=gen)
        chunks = int(((lens + 63) // 64).sum())
        assert chunks <= chunk_capacity(int(lens.sum()), n, 64)
    with pytest.raises(ValueError):
        chunk_capacity(-1, 1, 64)


def test_masks():
    import kda_b200

    x = torch.randn(1, 6, 3, requires_grad=True)
    cu = torch.tensor([0, 2, 4], dtype=torch.int32)
    mask = kda_b200.active_token_mask(x, cu)
    assert mask.tolist() == [True] * 4 + [False] * 2
    y = kda_b200.mask_inactive_tokens(x, mask)
    assert y[:, 4:].abs().max() == 0
    z = kda_b200.mask_inactive_token_gradients(x, mask)
    assert torch.equal(z, x)
    z.sum().backward()
    assert x.grad[:, :4].min() == 1 and x.grad[:, 4:].abs().max() == 0
    assert kda_b200.mask_inactive_tokens(x, None) is x


def test_profiler_range_is_free_without_a_profiler_and_named_under_one():
    """The reference's tracing mechanism (kda/utils.py:269-273): a null context when no torch
    profiler is active, a record_function range when one is."""
    import contextlib

    import torch
    from kda_b200 import _cabi

    assert isinstance(_cabi.profiler_range("kda_b200/x"), contextlib.nullcontext)
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU]) as prof:
        with _cabi.profiler_range("kda_b200/some_entry"):
            torch.ones(4).sum()
    assert any(e.name == "kda_b200/some_entry" for e in prof.events())
