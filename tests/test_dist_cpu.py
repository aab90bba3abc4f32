"""Host-side logic of the multi-GPU paths on CPU: sharding arithmetic, and the context-parallel
boundary-state chain run as two and three gloo ranks with the CPU oracle standing in for the
kernels (the protocol -- who sends what to whom, and the affine composition -- is what is tested)."""

import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_ranges_tile_the_grid():
    from kda_b200.dist import shard_ranges

    for batch, heads, world in [(8, 32, 1), (8, 32, 2), (8, 32, 4), (8, 32, 8), (1, 32, 8),
                                (2, 32, 8), (3, 8, 4)]:
        seen = torch.zeros(batch, heads, dtype=torch.int32)
        for rank in range(world):
            bs, hs = shard_ranges(batch, heads, world, rank)
            seen[bs, hs] += 1
        assert (seen == 1).all(), (batch, heads, world)
    with pytest.raises(ValueError):
        shard_ranges(3, 5, 4, 0)


class OracleSlice:
    """CPU stand-in with the interface of kda_b200.dist.CudaSlice."""

    def __init__(self, q, k, v, gate, beta):
        self.args = (q.double(), k.double(), v.double(), gate.double(), beta.double())

    def run(self, h_in):
        from oracle import kda_oracle as orc

        h = None if h_in is None else h_in.double()
        o, s = orc.chunk_kda_ref(*self.args, initial_state=h)
        return o, s.float()

    def zero_state_result(self):
        return self.run(None)[1]

    def transition(self):
        from oracle import kda_oracle as orc

        q, k, v, gate, beta = self.args
        per_token = gate.clone()
        t = gate.shape[1]
        for c0 in range(0, t, 64):
            per_token[:, c0 + 1:c0 + 64] = gate[:, c0 + 1:c0 + 64] - gate[:, c0:min(t, c0 + 64) - 1]
        return orc.slice_transition_ref(k[0], per_token[0], beta[0])[None].float()

    def slice_map(self):
        out, b = self.run(None)
        return out, b, self.transition(), None

    def correct(self, out, h_in, limit):
        return self.run(h_in)[0]

    def affine(self, trans, h_in, b):
        return trans @ h_in + b


def _cp_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "attention-gym_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from kda_b200.dist import cp_chunk_forward
        from oracle import kda_oracle as orc

        torch.set_num_threads(1)
        total = 64 * 2 * world + 40       # the last slice has a partial tail chunk
        inp = orc.make_inputs(1, total, 2, 16, 24, seed=21, with_state=True)
        lo = 128 * rank
        hi = total if rank + 1 == world else lo + 128
        sl = slice(lo, hi)
        out, h_out = cp_chunk_forward(inp["q"][:, sl], inp["k"][:, sl], inp["v"][:, sl],
                                      inp["cum_gate"][:, sl], inp["beta"][:, sl], inp["h0"],
                                      slice_factory=OracleSlice)
        ref_o, ref_s = orc.chunk_kda_ref(inp["q"].double(), inp["k"].double(), inp["v"].double(),
                                         inp["cum_gate"].double(), inp["beta"].double(),
                                         inp["h0"].double())
        err_o = float((out.double() - ref_o[:, sl]).abs().max())
        err_s = float((h_out.double() - ref_s).abs().max()) if rank + 1 == world else 0.0
        ret[rank] = (err_o, err_s)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_context_parallel_chain_gloo(world):
    port = 29600 + world + (os.getpid() % 200)
    with mp.Manager() as manager:
        ret = manager.dict()
        mp.spawn(_cp_worker, args=(world, port, ret), nprocs=world, join=True)
        for rank in range(world):
            err_o, err_s = ret[rank]
            assert err_o < 1e-5, f"rank {rank}: output error {err_o}"
            assert err_s < 1e-5, f"rank {rank}: final state error {err_s}"


def _oracle_slice_grads(q, k, v, gate, beta, h_in, d_out, dh_out):
    """CPU stand-in for kda_b200.dist.cuda_slice_grads: autograd through the fp64 oracle."""
    from oracle import kda_oracle as orc

    if h_in is None:
        h_in = torch.zeros(q.shape[0], q.shape[2], q.shape[3], v.shape[3])
    leaves = [t.detach().double().requires_grad_() for t in (q, k, v, gate, beta, h_in)]
    with torch.enable_grad():
        o, s = orc.chunk_kda_ref(*leaves[:5], initial_state=leaves[5])
        grads = torch.autograd.grad((o, s), leaves, (d_out.double(), dh_out.double()))
    return tuple(g.float() for g in grads)


def _cp_bwd_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "attention-gym_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from kda_b200.dist import _cp_forward, cp_chunk_backward
        from oracle import kda_oracle as orc

        torch.set_num_threads(1)
        total = 64 * 2 * world + 40
        inp = orc.make_inputs(1, total, 2, 16, 24, seed=22, with_state=True)
        gen = torch.Generator().manual_seed(5)
        d_out = torch.randn(inp["v"].shape, generator=gen)
        d_final = torch.randn(inp["h0"].shape, generator=gen)
        lo = 128 * rank
        hi = total if rank + 1 == world else lo + 128
        sl = slice(lo, hi)
        args = [inp[n][:, sl] for n in ("q", "k", "v", "cum_gate", "beta")]
        _, _, h_in, trans = _cp_forward(*args, inp["h0"], slice_factory=OracleSlice)
        grads = cp_chunk_backward(*args, h_in, trans, d_out[:, sl],
                                  d_final if rank + 1 == world else None,
                                  local_grads=_oracle_slice_grads)
        # the whole sequence on one rank
        leaves = [inp[n].double().requires_grad_() for n in ("q", "k", "v", "cum_gate", "beta", "h0")]
        o, s = orc.chunk_kda_ref(*leaves[:5], initial_state=leaves[5])
        ref = torch.autograd.grad((o, s), leaves, (d_out.double(), d_final.double()))
        errs = [float((g.double() - r[:, sl]).abs().max()) for g, r in zip(grads[:5], ref[:5])]
        if rank == 0:
            errs.append(float((grads[5].double() - ref[5]).abs().max()))
        ret[rank] = max(errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_context_parallel_backward_chain_gloo(world):
    """dq, dk, dv, d_gate, d_beta of every slice and d_initial_state on rank 0 equal the gradients
    of the unsplit sequence; only [H, K, V] state gradients cross ranks."""
    port = 29700 + world + (os.getpid() % 200)
    with mp.Manager() as manager:
        ret = manager.dict()
        mp.spawn(_cp_bwd_worker, args=(world, port, ret), nprocs=world, join=True)
        for rank in range(world):
            assert ret[rank] < 2e-5, f"rank {rank}: gradient error {ret[rank]}"


def _subgroup_worker(rank, world, port, ret):
    """World of 4 = two independent context-parallel groups of 2 (ranks {0, 1} and {2, 3})."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "attention-gym_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from kda_b200.dist import cp_chunk_forward
        from oracle import kda_oracle as orc

        torch.set_num_threads(1)
        groups = [dist.new_group([0, 1]), dist.new_group([2, 3])]
        mine = rank // 2
        local = rank % 2
        total = 64 * 2 * 2 + 17
        inp = orc.make_inputs(1, total, 2, 16, 24, seed=40 + mine, with_state=True)   # other data per group
        sl = slice(0, 128) if local == 0 else slice(128, total)
        out, h_out = cp_chunk_forward(inp["q"][:, sl], inp["k"][:, sl], inp["v"][:, sl],
                                      inp["cum_gate"][:, sl], inp["beta"][:, sl], inp["h0"],
                                      group=groups[mine], slice_factory=OracleSlice, timeout=60.0)
        ref_o, ref_s = orc.chunk_kda_ref(inp["q"].double(), inp["k"].double(), inp["v"].double(),
                                         inp["cum_gate"].double(), inp["beta"].double(),
                                         inp["h0"].double())
        err_o = float((out.double() - ref_o[:, sl]).abs().max())
        err_s = float((h_out.double() - ref_s).abs().max()) if local == 1 else 0.0
        ret[rank] = (err_o, err_s)
    finally:
        dist.destroy_process_group()


def test_context_parallel_chain_inside_subgroups_gloo():
    """Two context-parallel groups inside one world of four: boundary states must go to the
    neighbour inside the group (group-local ranks are translated to global ones)."""
    port = 29800 + (os.getpid() % 200)
    with mp.Manager() as manager:
        ret = manager.dict()
        mp.spawn(_subgroup_worker, args=(4, port, ret), nprocs=4, join=True)
        for rank in range(4):
            err_o, err_s = ret[rank]
            assert err_o < 1e-5 and err_s < 1e-5, f"rank {rank}: {err_o} {err_s}"


def _timeout_worker(rank, world, port, ret):
    """Rank 0 never sends its boundary state: rank 1 must give up with ChainTimeout instead of
    blocking forever."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "attention-gym_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import time

    from kda_b200.dist import ChainTimeout, cp_chunk_forward
    from oracle import kda_oracle as orc

    torch.set_num_threads(1)
    inp = orc.make_inputs(1, 192, 1, 16, 24, seed=50)
    if rank == 0:
        time.sleep(4.0)                                      # a rank that hangs before its send
        ret[0] = "idle"
    else:
        sl = slice(128, 192)
        t0 = time.monotonic()
        try:
            cp_chunk_forward(inp["q"][:, sl], inp["k"][:, sl], inp["v"][:, sl],
                             inp["cum_gate"][:, sl], inp["beta"][:, sl], None,
                             slice_factory=OracleSlice, timeout=1.0)
            ret[1] = "no timeout"
        except ChainTimeout as exc:
            ret[1] = (time.monotonic() - t0, str(exc))
    os._exit(0)      # the timed-out gloo pair is closed: no collective tear-down


def test_chain_receive_has_a_host_deadline_gloo():
    port = 29850 + (os.getpid() % 100)
    with mp.Manager() as manager:
        ret = manager.dict()
        mp.spawn(_timeout_worker, args=(2, port, ret), nprocs=2, join=True)
        assert ret[0] == "idle"
        waited, message = ret[1]
        assert 0.9 <= waited < 3.5, waited
        assert "no boundary state from rank 0" in message
