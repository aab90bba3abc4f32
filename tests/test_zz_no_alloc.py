"""The allocation-free chunked forward, kda_chunk_fwd_noalloc.

It exists for hosts that cannot allocate device memory while they run -- for example an inference
server whose own memory pool already holds the whole GPU -- and keeps its scratch in a static
device array inside the library.  The test drives it through the C ABI (ctypes), exactly as such
a host would, and checks it against kda_chunk_fwd on two calls in a row: the second call uses
different inputs, so anything left in the shared scratch by the first call would show.  Both entry
points run the same kernels on the same values, so their results must agree bit for bit.  The
second call must also leave the amount of free device memory unchanged: the first call on a device
is the one that makes CUDA load the module holding the array, later ones claim nothing.
This file is collected last on purpose: if it fails, every other test has already run.
"""

import pytest
import torch

from kda_b200 import _cabi
from kda_b200.chunk_schedule import prepare_ragged_chunk_metadata
from oracle import kda_oracle as orc
from helpers import assert_normalised

pytestmark = pytest.mark.gpu
TOL = 2e-2  # normalised max error, the tolerance of the other bf16 chunk tests


def _buffers(tokens, heads, nseq, dev):
    return dict(
        out=torch.zeros(1, tokens, heads, 128, dtype=torch.bfloat16, device=dev),
        aqk=torch.zeros(1, tokens, heads, 64, dtype=torch.bfloat16, device=dev),
        akk=torch.zeros(1, tokens, heads, 64, dtype=torch.bfloat16, device=dev),
        state=torch.zeros(nseq, heads, 128, 128, dtype=torch.float32, device=dev),
    )


def _run_pair(seed, lengths, tokens, heads, check_memory=False):
    dev = torch.device("cuda")
    inp = orc.make_inputs(1, tokens, heads, 128, 128, seed=seed, with_state=True, lengths=lengths)
    q, k, v = (inp[n].bfloat16().to(dev) for n in ("q", "k", "v"))
    g, beta, h0 = inp["cum_gate"].to(dev), inp["beta"].to(dev), inp["h0"].to(dev)
    meta = prepare_ragged_chunk_metadata(inp["cu_seqlens"].to(dev), tokens, 64)
    nseq = len(lengths)
    lib, p, stream = _cabi.lib(), _cabi.ptr, _cabi.stream()
    ref, got = _buffers(tokens, heads, nseq, dev), _buffers(tokens, heads, nseq, dev)
    nbytes = lib.kda_chunk_fwd_workspace_bytes(tokens, heads)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    common = (p(q), p(k), p(v), p(g), p(beta), p(h0))
    tail = (p(meta.cu_seqlens), p(meta.chunk_offsets), nseq, tokens, heads, 128, 128, meta.capacity)
    rc = lib.kda_chunk_fwd(*common, p(ref["state"]), p(ref["out"]), p(ref["aqk"]), p(ref["akk"]),
                           *tail, p(ws), nbytes, stream)
    assert rc == 0
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = lib.kda_chunk_fwd_noalloc(*common, p(got["state"]), p(got["out"]), p(got["aqk"]),
                                   p(got["akk"]), *tail, stream)
    assert rc == 0
    torch.cuda.synchronize()
    if check_memory:
        assert torch.cuda.mem_get_info()[0] == free_before, "the no-alloc entry point took device memory"
    active = int(inp["cu_seqlens"][-1])
    for name in ("out", "aqk", "akk"):
        assert torch.equal(got[name][:, :active], ref[name][:, :active]), name
    assert torch.equal(got["state"], ref["state"]), "state"
    oracle_o, oracle_s = orc.chunk_kda_ref(inp["q"].bfloat16().float(), inp["k"].bfloat16().float(),
                                           inp["v"].bfloat16().float(), inp["cum_gate"],
                                           inp["beta"], inp["h0"], inp["cu_seqlens"])
    assert_normalised(got["out"][:, :active].float(), oracle_o[:, :active], TOL, "out vs oracle")
    assert_normalised(got["state"], oracle_s, TOL, "state vs oracle")


def test_noalloc_matches_workspace_entry_point_twice():
    _run_pair(seed=41, lengths=[130, 64, 0, 90], tokens=300, heads=2)
    # second call, other shapes and data; the module with the array is loaded by now
    _run_pair(seed=42, lengths=[50, 200], tokens=256, heads=4, check_memory=True)


def test_noalloc_rejects_oversized_problems():
    lib = _cabi.lib()
    # 1 Ki bytes of scratch per (token, head): 32 MiB holds 32768 of them
    t = torch.zeros(8, device="cuda")
    args = [_cabi.ptr(t)] * 12
    rc = lib.kda_chunk_fwd_noalloc(*args, 1, 32768 + 64, 1, 128, 128, 600, _cabi.stream())
    assert rc == -4
