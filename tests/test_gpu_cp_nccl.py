"""Context-parallel forward and backward over a real NCCL point-to-point chain: one process per
GPU, the only traffic is the fp32 boundary state [H, 128, 128] from rank r to rank r + 1 and, in
backward, its gradient from rank r + 1 to rank r.  Needs at least two
GPUs (skipped otherwise); the single-process emulation in test_gpu_cp.py covers the same code on
one GPU."""

import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, total, heads, out_dir):
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for p in (root, os.path.join(root, "attention-gym_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist
    import kda_b200
    from kda_b200.dist import cp_chunk_forward, cp_chunk_kda
    from oracle import kda_oracle as orc

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    inp = orc.make_inputs(1, total, heads, 128, 128, seed=41, with_state=True)   # same on every rank
    per = (total // world) // 64 * 64
    lo, hi = rank * per, (total if rank + 1 == world else (rank + 1) * per)
    dev = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inp.items()}
    q, k, v = (dev[n][:, lo:hi].bfloat16() for n in ("q", "k", "v"))
    o, s = cp_chunk_forward(q, k, v, dev["cum_gate"][:, lo:hi], dev["beta"][:, lo:hi], dev["h0"])
    # differentiable variant: forward chain, then the state-gradient chain in backward
    gen = torch.Generator().manual_seed(8)
    d_out = torch.randn(inp["v"].shape, generator=gen).bfloat16().cuda()
    d_final = torch.randn(inp["h0"].shape, generator=gen).cuda()
    leaves = [t.clone().requires_grad_() for t in
              (q, k, v, dev["cum_gate"][:, lo:hi], dev["beta"][:, lo:hi], dev["h0"])]
    o2, s2 = cp_chunk_kda(*leaves)
    grads = torch.autograd.grad((o2, s2), leaves, (d_out[:, lo:hi], d_final), allow_unused=True)
    torch.save({"o": o.cpu(), "s": s.cpu(), "o2": o2.detach().cpu(), "lo": lo, "hi": hi,
                "grads": [None if g is None else g.cpu() for g in grads]},
               os.path.join(out_dir, f"r{rank}.pt"))
    if rank == 0:
        full = [t.clone().requires_grad_() for t in
                (dev["q"].bfloat16(), dev["k"].bfloat16(), dev["v"].bfloat16(), dev["cum_gate"],
                 dev["beta"], dev["h0"])]
        fo, fs = kda_b200.chunk_kda(*full, output_final_state=True)
        fg = torch.autograd.grad((fo, fs), full, (d_out, d_final))
        torch.save({"o": fo.detach().cpu(), "s": fs.detach().cpu(), "grads": [g.cpu() for g in fg]},
                   os.path.join(out_dir, "full.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_cp_chain_over_nccl(tmp_path):
    import torch.multiprocessing as mp

    from helpers import assert_normalised

    world = min(torch.cuda.device_count(), 4)
    total, heads = 64 * 4 * world + 37, 4
    mp.spawn(_worker, args=(world, 29541, total, heads, str(tmp_path)), nprocs=world, join=True)
    full = torch.load(tmp_path / "full.pt")
    parts = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    out = torch.cat([p["o"] for p in parts], 1)
    assert out.shape == full["o"].shape
    assert_normalised(out.float(), full["o"].float(), 2e-2, "NCCL chain output vs single GPU")
    assert_normalised(parts[-1]["s"], full["s"], 2e-2, "NCCL chain final state vs single GPU")
    assert_normalised(torch.cat([p["o2"] for p in parts], 1).float(), full["o"].float(), 2e-2,
                      "differentiable chain output vs single GPU")
    for i, name in enumerate(("dq", "dk", "dv", "d_gate", "d_beta")):
        got = torch.cat([p["grads"][i] for p in parts], 1)
        assert_normalised(got.float(), full["grads"][i].float(), 2e-2, f"NCCL chain {name} vs single GPU")
    assert_normalised(parts[0]["grads"][5], full["grads"][5], 2e-2,
                      "NCCL chain d_initial_state vs single GPU")
