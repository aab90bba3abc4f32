"""Benchmark of the KDA hot path: chunked forward + backward tokens/s (H32, K=V=128, bf16).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--small]

One step = one forward + backward pass of ``chunk_kda`` over one batch of synthetic input with the
shapes and value distributions of the headline configuration (B=8, T=4096, H=32, K=V=128,
chunk 64; q, k L2-normalised N(0,1), v ~ N(0,1), g = logsigmoid(N(0,1)), beta = sigmoid(N(0,1)),
dO ~ N(0,1)).  Inputs (1.5 GiB) are far larger than L2, so no flush is needed between steps.

Rank 0 prints one JSON line.  ``value`` is device-resident throughput (CUDA events, max over
ranks, per-kernel event recording switched off); ``e2e`` is the same step with pinned HOST buffers,
host<->device copies inside the timed region; ``kernels`` / ``roofline`` come from a second pass of
the same steps with the library's per-kernel CUDA events on the launching stream switched on
(``roofline`` describes the kernel with the largest share); ``cpu_baseline`` is the CPU
implementation of the path timed on a bounded sample on this machine's cores.  Multi-GPU runs shard
by (batch, head) with no collective: every rank runs the full per-GPU workload (weak scaling).
Two more sub-objects measure the splits of a fixed amount of work over the N GPUs:
``strong`` = the single B=8 batch of the headline configuration cut by (batch, head) with
``shard_ranges`` (no collective), ``cp`` = one sequence of 1,048,576 tokens, forward, cut into N
contiguous slices whose boundary states travel along an NCCL point-to-point chain
(``cp_chunk_forward``), with a self-check against a single-GPU run on rank 0.

``--impl reference`` times the reference's own CPU code for the path when ``oracle/_ref`` holds it
(see oracle/build_ref.py), else the CPU port (the oracle).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "attention-gym_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

METRIC = "KDA fwd+bwd tokens/s (H32,K=V=128,bf16)"
H, D, CHUNK = 32, 128, 64
LOG2E = 1.4426950408889634

# algorithmic HBM bytes per (token, head) of each kernel: what its interface must read + write
STAGE_BYTES = {
    # q,k,v bf16 + G fp32 + beta -> Aqk, Akk, w, u, kg, qg
    "prepare": 3 * 256 + 512 + 4 + 2 * 128 + 4 * 256,
    "state_fwd": 4 * 256 + 128 + 8 + 256,                       # w,u,kg,qg,Aqk,G_last -> o
    "state_fwd_recompute": 4 * 256 + 128 + 8 + 256 + 512 + 256, # ... -> o, h[c] (bf16) and v_new (kept)
    "state_bwd": 3 * 256 + 256 + 128 + 8 + 512 + 256,           # w,kg,qg,dO,Aqk -> dh[c], dv2
    # h, dh (bf16 [128,128] per chunk = 512 B per token each), dO, v_new, dv2, v, k, q, G, Akk, beta
    # -> dq, dk, dv, dG, dbeta
    "bwd_chunk": 1024 + 6 * 256 + 512 + 128 + 4 + 3 * 256 + 512 + 4,
}
# DRAM bytes per (token, head) and launch that ncu measured (dram__bytes_read + dram__bytes_write on
# the B=2 case, which grows in proportion to the units; see profiles/)
NCU_TRAFFIC = {"bwd_chunk": 4370, "state_fwd": 2018, "state_bwd": 1780, "prepare": 2383}
# algorithmic FLOP per (token, head) of each kernel (dense 64-wide tiles, no causal discount;
# P = 2*64*128 = 16384, S = 2*128*128 = 32768); they add up to PATH_FLOP_FWD_BWD
STAGE_FLOP = {
    "prepare": 4 * 16384 + 2731,            # K~K~^T, Q~K~^T, w, u + the triangular solve
    "state_fwd": 3 * 32768 + 16384,         # w h, kg^T v_new, qg h + Aqk v_new
    "state_bwd": 3 * 32768 + 16384,         # kg dh, qg^T dO, w^T dv2 + Aqk^T dO
    "bwd_chunk": 3 * 32768 + 16384 + 4 * 16384 + 16384 + 5 * 16384,
}
# the path's algorithmic minimum (inputs once, outputs once), bytes per token per head
PATH_BYTES_FWD_BWD = 4620
PATH_FLOP_FWD_BWD = 576171


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None
        self.window = None          # (t0, t1) of the timed region, time.monotonic()

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append((time.monotonic(), parts))

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def mark(self, t0, t1):
        self.window = (t0, t1)

    def summary(self):
        # samples taken inside the timed region; a region shorter than the sampling period widens
        # the window by 100 ms on both sides (the same kernels run in the warm-up before it)
        picked = self.samples
        if self.window is not None:
            t0, t1 = self.window
            picked = [s for s in self.samples if t0 <= s[0] <= t1]
            if not picked:
                picked = [s for s in self.samples if t0 - 0.1 <= s[0] <= t1 + 0.1]
        picked = [s[1] for s in picked]
        if not picked:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        return self._summarise(picked)

    @staticmethod
    def _summarise(samples):
        mhz = sorted(int(s[0]) for s in samples if s[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in samples)]
        mx = [int(s[1]) for s in samples if s[1].isdigit()]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(samples)}


def make_host_inputs(batch, tokens, seed, pin):
    """Synthetic step inputs on the host (pinned when asked), in the dtypes the kernels consume."""

    gen = torch.Generator().manual_seed(seed)
    shape = (batch, tokens, H, D)

    def rnd(*s):
        return torch.randn(*s, generator=gen)

    q = torch.nn.functional.normalize(rnd(*shape), dim=-1).bfloat16()
    k = torch.nn.functional.normalize(rnd(*shape), dim=-1).bfloat16()
    v = rnd(*shape).bfloat16()
    g = torch.nn.functional.logsigmoid(rnd(*shape)) * LOG2E
    g = g.view(batch, tokens // CHUNK, CHUNK, H, D).cumsum(2).view(shape).contiguous()
    beta = torch.sigmoid(rnd(batch, tokens, H))
    do = rnd(*shape).bfloat16()
    out = {"q": q, "k": k, "v": v, "g": g, "beta": beta, "do": do}
    if pin:
        out = {n: t.pin_memory() for n, t in out.items()}
    return out


def step_device(kda_b200, dev):
    q, k, v, g, beta = (dev[n].detach().requires_grad_(True) for n in ("q", "k", "v", "g", "beta"))
    o, _ = kda_b200.chunk_kda(q, k, v, g, beta)
    grads = torch.autograd.grad(o, (q, k, v, g, beta), dev["do"])
    return o, grads


def run_ours(args):
    import kda_b200
    from kda_b200 import _cabi

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    batch, tokens = (2, 4096) if args.small else (8, 4096)
    tokens_per_step = batch * tokens
    host = make_host_inputs(batch, tokens, seed=1234 + rank, pin=True)
    dev = {n: t.to(device, non_blocking=True) for n, t in host.items()}
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # the sampler starts before the warm-up so that nvidia-smi is already reporting when the timed
    # region begins; only samples whose timestamps fall inside the region are summarised
    with ClockSampler(local_rank) as clocks:
        for _ in range(args.warmup):
            step_device(kda_b200, dev)
        for _ in range(30):                      # keep the GPU under the same load until samples arrive
            if clocks.samples:
                break
            step_device(kda_b200, dev)
            torch.cuda.synchronize()
        barrier()
        _cabi.stage_timing(False)
        launches0 = _cabi.launch_count
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t_begin = time.monotonic()
        start.record()
        for _ in range(args.steps):
            step_device(kda_b200, dev)
        stop.record()
        barrier()
        clocks.mark(t_begin, time.monotonic())
    ms = start.elapsed_time(stop)
    launches = _cabi.launch_count - launches0
    # per-kernel breakdown: the same steps once more with the library's event pairs switched on
    _cabi.read_stage_timing(reset=True)
    _cabi.stage_timing(True)
    for _ in range(args.steps):
        step_device(kda_b200, dev)
    torch.cuda.synchronize()
    stages = _cabi.read_stage_timing(reset=True)
    _cabi.stage_timing(False)

    decode = None if args.skip_decode else bench_decode(kda_b200, _cabi, device, load_peaks())
    preops = None if (args.skip_decode or rank != 0) else bench_preops(device, load_peaks(), batch, tokens)
    norm_fusion = None if (args.skip_decode or rank != 0) else bench_layer_norm_fusion(kda_b200, device, batch, tokens)
    layer = None if (args.skip_decode or rank != 0) else bench_layer(kda_b200, _cabi, device)
    others = None
    if args.other_configs and rank == 0:
        del dev
        torch.cuda.empty_cache()
        others = bench_other_configs(kda_b200, _cabi, device)
        dev = {n: t.to(device, non_blocking=True) for n, t in host.items()}
    # ---- end to end: pinned host buffers in, pinned host buffers out, every copy inside the timed
    # region.  Three streams (H2D, compute, D2H) with double-buffered device inputs and host
    # outputs, so the copies of neighbouring steps overlap the kernels the way a host-buffer caller
    # of the library would drive it.
    e2e_steps = 0 if args.skip_e2e else max(1, args.steps)
    ms_e2e, h2d, d2h = float("nan"), 0, 0
    if e2e_steps:
        s_in, s_out, s_main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
        dev_in = [{n: torch.empty_like(t, device=device) for n, t in host.items()} for _ in range(2)]
        host_out = [None, None]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

        def run_e2e(n):
            for i in range(n):
                b = i & 1
                with torch.cuda.stream(s_in):
                    if i >= 2:
                        s_in.wait_event(ev_done[b])        # device inputs of step i-2 consumed
                    for name, t in host.items():
                        dev_in[b][name].copy_(t, non_blocking=True)
                    ev_in[b].record(s_in)
                s_main.wait_event(ev_in[b])
                o, grads = step_device(kda_b200, dev_in[b])
                outs = (o,) + tuple(grads)
                ev_done[b].record(s_main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[b])
                    if host_out[b] is None:
                        host_out[b] = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in outs]
                    elif i >= 2:
                        ev_out[b].synchronize()           # host buffers of step i-2 are free again
                    for h, t in zip(host_out[b], outs):
                        t.record_stream(s_out)
                        h.copy_(t, non_blocking=True)
                    ev_out[b].record(s_out)

        run_e2e(2)
        barrier()
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s2.record(s_main)
        s_in.wait_event(s2)
        run_e2e(e2e_steps)
        s_main.wait_stream(s_out)
        e2.record(s_main)
        barrier()
        ms_e2e = s2.elapsed_time(e2)
        h2d = sum(t.numel() * t.element_size() for t in host.values())
        d2h = sum(t.numel() * t.element_size() for t in host_out[0])

    if world > 1:
        t = torch.tensor([ms, ms_e2e], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
    strong = cp = None
    if not args.skip_splits:
        del dev
        if e2e_steps:
            del dev_in, host_out
        torch.cuda.empty_cache()
        strong = bench_strong(kda_b200, device, rank, world, args.steps, args.warmup, barrier)
        torch.cuda.empty_cache()
        cp = bench_cp(kda_b200, _cabi, device, rank, world, barrier, tokens=args.cp_tokens)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    value = world * tokens_per_step * args.steps / (ms * 1e-3)
    e2e_value = world * tokens_per_step * e2e_steps / (ms_e2e * 1e-3) if e2e_steps else 0.0
    # dominant kernel = largest share of the timed region
    roofline, breakdown = None, {}
    total_stage_ms = sum(v[1] for v in stages.values()) or 1.0
    for name, (n, tot) in stages.items():
        sec = tot / n * 1e-3
        units_ = tokens_per_step * H
        b_unit = STAGE_BYTES["state_fwd_recompute"] if name == "state_fwd" else STAGE_BYTES.get(name, 0)
        breakdown[name] = {"launches": n, "ms_per_launch": round(tot / n, 4),
                           "share": round(tot / total_stage_ms, 4),
                           "algorithmic_gbs": round(b_unit * units_ / sec / 1e9, 1),
                           "algorithmic_tflops": round(STAGE_FLOP.get(name, 0) * units_ / sec / 1e12, 1)}
    if stages:
        top = max(stages, key=lambda n: stages[n][1])
        n, tot = stages[top]
        per_launch_ms = tot / n
        units = tokens_per_step * H
        key = top
        # the default path keeps the forward intermediates: state_fwd also writes h[c] and v_new
        per_unit = STAGE_BYTES["state_fwd_recompute"] if top == "state_fwd" else STAGE_BYTES.get(key, 0)
        achieved = per_unit * units / (per_launch_ms * 1e-3) / 1e9
        roofline = {"kernel": top, "bound": "hbm", "achieved": round(achieved, 1),
                    "peak": peaks["hbm_gbs"], "peak_source": peaks["source"], "unit": "GB/s",
                    "frac": round(achieved / peaks["hbm_gbs"], 4),
                    "traffic": NCU_TRAFFIC[top] * units if top in NCU_TRAFFIC else None,
                    "traffic_source": ("ncu dram__bytes_read.sum + dram__bytes_write.sum of one capture of "
                                       "the B=2 case (profiles/), scaled by the units of this launch; "
                                       "not measured in this run") if top in NCU_TRAFFIC else None,
                    "bytes_per_token_head": per_unit, "ms_per_launch": round(per_launch_ms, 4)}
    path = {"hbm_frac": round(value * H * PATH_BYTES_FWD_BWD / 1e9 / world / peaks["hbm_gbs"], 4),
            "tensor_frac": round(value * H * PATH_FLOP_FWD_BWD / 1e12 / world / peaks["bf16_tflops"], 4),
            "achieved_gbs": round(value * H * PATH_BYTES_FWD_BWD / 1e9 / world, 1),
            "achieved_tflops": round(value * H * PATH_FLOP_FWD_BWD / 1e12 / world, 1)}
    cpu = None if args.skip_cpu else cpu_baseline(bounded=True)
    line = {
        "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"config1: chunk_kda fwd+bwd B={batch} T={tokens} H={H} K=V={D} "
                               f"chunk={CHUNK} per GPU, sharded by (batch, head), no collective",
                   "l2": "inputs (1.5 GiB) larger than L2, no flush"},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": e2e_steps},
        "gpu_launches": launches,
        "clocks": clocks.summary(),
        "roofline": roofline,
        "path_roofline": path,
        "kernels": breakdown,
        "cpu_baseline": cpu,
        "decode": decode,
        "preops": preops,
        "layer_qk_norm": norm_fusion,
        "layer": layer,
        "other_configs": others,
        "strong": strong,
        "cp": cp,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _max_over_ranks(values, device, world):
    if world == 1:
        return [float(v) for v in values]
    import torch.distributed as dist

    t = torch.tensor(values, device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]


def _all_ranks(values, device, world):
    """[world][len(values)] list: every rank's row."""
    t = torch.tensor(values, device=device, dtype=torch.float64)
    if world == 1:
        return [t.tolist()]
    import torch.distributed as dist

    rows = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(rows, t)
    return [r.tolist() for r in rows]


def bench_strong(kda_b200, device, rank, world, steps, warmup, barrier):
    """Strong scaling of the headline step: ONE batch of B=8 rows (config 1) cut over the ranks by
    (batch, head) with shard_ranges; no collective on the data path.  Row r of the batch comes from
    seed 9000 + r whatever the number of ranks, so every N works on the same global batch."""
    from kda_b200.dist import shard_ranges

    rows, heads = shard_ranges(8, H, world, rank)
    parts = [_device_inputs(1, 4096, device, 9000 + r) for r in range(8)[rows]]
    dev = {n: torch.cat([p[n] for p in parts], 0)[:, :, heads].contiguous() for n in parts[0]}
    del parts
    for _ in range(max(warmup, 3)):
        step_device(kda_b200, dev)
    barrier()
    a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        step_device(kda_b200, dev)
    z.record()
    barrier()
    (ms,) = _max_over_ranks([a.elapsed_time(z)], device, world)
    shape = dev["q"].shape
    return {"workload": f"config1, one batch B=8 T=4096 H={H} fwd+bwd cut by (batch, head) over {world} "
                        f"GPU(s): B={shape[0]} H={shape[2]} per GPU, no collective",
            "scaling": "strong", "ms_per_step": round(ms / steps, 4),
            "tokens_per_s": round(8 * 4096 * steps / (ms * 1e-3), 1)}


def bench_cp(kda_b200, _cabi, device, rank, world, barrier, tokens=1 << 20, iters=3):
    """Context parallelism (config 4): one sequence of `tokens` tokens, forward, in `world` contiguous
    slices; only the fp32 boundary state [H, 128, 128] crosses GPUs, along an NCCL point-to-point
    chain.  With one GPU this is the plain forward.  Includes a self-check: two reduced sequences
    (65,536 tokens; the benchmark's forgetful gates, and gates scaled by 0.02 so that the slice
    transitions stay dense) go through the same chain and the last rank's outputs and the final
    state are compared on rank 0 with its own single-GPU pass over the whole sequence."""
    from kda_b200.dist import cp_chunk_forward

    per = tokens // world
    if per % CHUNK:
        raise SystemExit("slices must hold whole chunks")

    def forward(d):
        with torch.no_grad():
            if world == 1:
                return kda_b200.chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], output_final_state=True)
            return cp_chunk_forward(d["q"], d["k"], d["v"], d["g"], d["beta"], None, timeout=120.0)

    d = _device_inputs(1, per, device, 9100 + rank, with_do=False)
    for _ in range(2):
        forward(d)
    barrier()
    a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        forward(d)
    z.record()
    barrier()
    (ms,) = _max_over_ranks([a.elapsed_time(z)], device, world)
    _cabi.read_stage_timing(reset=True)
    _cabi.stage_timing(True)
    forward(d)
    torch.cuda.synchronize()
    st = _cabi.read_stage_timing(reset=True)
    _cabi.stage_timing(False)
    per_rank = _all_ranks([st.get("prepare", (0, 0.0))[1], st.get("state_fwd", (0, 0.0))[1],
                           st.get("state_fwd", (0, 0.0))[0]], device, world)
    del d
    torch.cuda.empty_cache()

    # ---- self-check on reduced sequences
    check = {}
    small = 65536 // world
    for name, scale in (("forgetful_gates", 1.0), ("mild_gates", 0.02)):
        mine = _device_inputs(1, small, device, 9200 + rank, with_do=False)
        mine["g"] = mine["g"] * scale
        o, s = forward(mine)
        if world == 1:
            check[name] = "single GPU: nothing to compare"
            continue
        import torch.distributed as dist

        if rank == world - 1:
            dist.send(o.contiguous(), 0)
            dist.send(s.contiguous(), 0)
        if rank == 0:
            o_last, s_last = torch.empty_like(o), torch.empty_like(s)
            dist.recv(o_last, world - 1)
            dist.recv(s_last, world - 1)
            parts = [_device_inputs(1, small, device, 9200 + r, with_do=False) for r in range(world)]
            whole = {n: torch.cat([p[n] for p in parts], 1) for n in parts[0]}
            whole["g"] = whole["g"] * scale
            with torch.no_grad():
                ro, rs = kda_b200.chunk_kda(whole["q"], whole["k"], whole["v"], whole["g"], whole["beta"],
                                            output_final_state=True)
            ro = ro[:, -small:].float()
            check[name] = {
                "output_last_slice": float((o_last.float() - ro).abs().max() / ro.abs().max()),
                "final_state": float((s_last - rs).abs().max() / rs.abs().max())}
            del parts, whole
        del mine
        torch.cuda.empty_cache()
    if rank == 0 and world > 1:
        check["tolerance"] = 2e-2
        check["ok"] = all(v <= 2e-2 for c in check.values() if isinstance(c, dict) for v in c.values())
    return {"workload": f"config4: one sequence of {tokens} tokens, H{H}, forward with final state, "
                        f"{world} contiguous slice(s); boundary states over an NCCL point-to-point chain",
            "scaling": "strong", "ms_per_step": round(ms / iters, 3),
            "tokens_per_s": round(tokens * iters / (ms * 1e-3), 1),
            "per_rank_ms": {"prepare": [round(r[0], 3) for r in per_rank],
                            "state_fwd": [round(r[1], 3) for r in per_rank],
                            "state_fwd_launches": [int(r[2]) for r in per_rank]},
            "check": check}


def bench_layer_norm_fusion(kda_b200, device, batch=8, tokens=4096, iters=10):
    """The q / k L2 normalisation of the layer at the headline shapes, fwd+bwd: as the two separate
    l2norm launches of the reference before the core (and two more after it in backward), against
    chunk_kda(normalize_qk=True), which normalises inside its first forward and last backward
    kernel.  Same unnormalised q, k in both arms; CUDA events."""
    d = _device_inputs(batch, tokens, device, 9300)
    gen = torch.Generator(device=device).manual_seed(9301)
    d["q"] = (d["q"].float() * (0.5 + 3 * torch.rand(batch, tokens, H, 1, generator=gen, device=device))).bfloat16()
    d["k"] = (d["k"].float() * (0.5 + 3 * torch.rand(batch, tokens, H, 1, generator=gen, device=device))).bfloat16()

    def step(fused):
        q, k, v, g, beta = (d[n].detach().requires_grad_(True) for n in ("q", "k", "v", "g", "beta"))
        if fused:
            o, _ = kda_b200.chunk_kda(q, k, v, g, beta, normalize_qk=True)
        else:
            o, _ = kda_b200.chunk_kda(kda_b200.l2norm(q), kda_b200.l2norm(k), v, g, beta)
        return torch.autograd.grad(o, (q, k, v, g, beta), d["do"])

    out = {}
    for name, fused in (("separate_l2norm_launches", False), ("normalisation_inside_the_core", True)):
        for _ in range(3):
            step(fused)
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(iters):
            step(fused)
        z.record()
        torch.cuda.synchronize()
        out[name] = {"ms_per_step": round(a.elapsed_time(z) / iters, 4)}
    out["workload"] = f"l2norm(q), l2norm(k) + chunk_kda fwd+bwd, B={batch} T={tokens} H={H}"
    return out


def bench_layer(kda_b200, _cabi, device, batch=2, tokens=4096, hidden=4096, iters=5):
    """One KDAAttention layer (the reference example's module on these kernels), forward + backward
    at H=32, head 128: ms per step and how it splits between this library's kernels (CUDA-event
    pairs of the library) and everything else (the cuBLAS projections, casts, masks)."""
    torch.manual_seed(11)
    layer = kda_b200.KDAAttention(hidden, H, D, backend="fused", device=device)
    x = torch.randn(batch, tokens, hidden, device=device, dtype=torch.bfloat16, requires_grad=True)
    params = list(layer.parameters())

    def step():
        out = layer(x).hidden_states
        return torch.autograd.grad(out, [x] + params, torch.ones_like(out))

    for _ in range(2):
        step()
    torch.cuda.synchronize()
    a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        step()
    z.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(z) / iters
    _cabi.read_stage_timing(reset=True)
    _cabi.stage_timing(True)
    step()
    torch.cuda.synchronize()
    stages = _cabi.read_stage_timing(reset=True)
    _cabi.stage_timing(False)
    ours = sum(v[1] for v in stages.values())
    return {"workload": f"KDAAttention fwd+bwd, B={batch} T={tokens} hidden={hidden} H={H} head={D}, bf16",
            "ms_per_step": round(ms, 3), "tokens_per_s": round(batch * tokens / (ms * 1e-3), 1),
            "ms_in_this_librarys_kernels": round(ours, 3),
            "kernels_ms": {k: round(v[1], 3) for k, v in stages.items()}}


def bench_decode(kda_b200, _cabi, device, peaks, nseq=256, steps=200):
    """Recurrent decode step (256 sequences, H32, K=V=128, fp32 state, bf16 tokens): us per step and
    achieved HBM bandwidth of the state read-modify-write (2 * 64 KiB per (sequence, head))."""
    gen = torch.Generator().manual_seed(5)
    state = (0.02 * torch.randn(nseq, H, D, D, generator=gen)).to(device)
    ins = []
    for _ in range(4):
        q = torch.nn.functional.normalize(torch.randn(nseq, 1, H, D, generator=gen), dim=-1)
        k = torch.nn.functional.normalize(torch.randn(nseq, 1, H, D, generator=gen), dim=-1)
        v = torch.randn(nseq, 1, H, D, generator=gen)
        g = torch.nn.functional.logsigmoid(torch.randn(nseq, 1, H, D, generator=gen)) * 1.4426950408889634
        b = torch.sigmoid(torch.randn(nseq, 1, H, generator=gen))
        ins.append(tuple(t.bfloat16().to(device) for t in (q, k, v, g, b)))
    idx = torch.arange(1, nseq + 1, dtype=torch.int32, device=device)
    pool = torch.cat((torch.zeros_like(state[:1]), state), 0)  # slot 0 is the padding slot

    def step(i):
        q, k, v, g, b = ins[i % 4]
        return kda_b200.recurrent_kda(q, k, v, g, b, pool, state_indices=idx)[0]

    for i in range(5):
        step(i)
    torch.cuda.synchronize()
    _cabi.read_stage_timing(reset=True)
    _cabi.stage_timing(True)
    a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        step(i)
    z.record()
    torch.cuda.synchronize()
    kern = _cabi.read_stage_timing(reset=True).get("recurrent", (0, 0.0))
    _cabi.stage_timing(False)
    us = a.elapsed_time(z) * 1e3 / steps
    kernel_us = kern[1] * 1e3 / max(kern[0], 1)
    bytes_per_step = nseq * H * (2 * D * D * 4 + 3 * D * 2 + 2 * D * 2 + 2)
    gbs = bytes_per_step / (kernel_us * 1e-6) / 1e9
    # the whole serving step: projection rows -> conv decode + SiLU + l2norm + gate (one kernel),
    # then the state update (second kernel)
    c = 3 * H * D
    weight = (0.5 * torch.randn(c, 4, generator=gen)).bfloat16().to(device)
    conv_pool = torch.randn(nseq + 1, 3, c, generator=gen).bfloat16().to(device)
    a_log = (0.1 * torch.randn(H, generator=gen)).to(device)
    dt_bias = (0.1 * torch.randn(H, D, generator=gen)).to(device)
    xs = [torch.randn(nseq, c, generator=gen).bfloat16().to(device) for _ in range(4)]
    raws = [torch.randn(nseq, H, D, generator=gen).bfloat16().to(device) for _ in range(4)]
    betas = [ins[i][4].reshape(nseq, H) for i in range(4)]

    def full_step(i):
        return kda_b200.decode_step(xs[i % 4], weight, conv_pool, raws[i % 4], a_log, dt_bias,
                                    betas[i % 4], pool, idx)

    for i in range(5):
        full_step(i)
    torch.cuda.synchronize()
    a.record()
    for i in range(steps):
        full_step(i)
    z.record()
    torch.cuda.synchronize()
    full_us = a.elapsed_time(z) * 1e3 / steps
    # the same step replayed from a CUDA graph (how a serving loop drives it: no host work per token)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        full_step(0)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        full_step(0)
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize()
    a.record()
    for _ in range(steps):
        graph.replay()
    z.record()
    torch.cuda.synchronize()
    graph_us = a.elapsed_time(z) * 1e3 / steps
    return {"workload": f"config3: {nseq} sequences x H{H}, K=V={D}, paged fp32 state, bf16 tokens",
            "us_per_step": round(us, 2), "kernel_us": round(kernel_us, 2),
            "tokens_per_s": round(nseq / (us * 1e-6), 1),
            "decode_step_with_preprocessing_us": round(full_us, 2),
            "decode_step_graph_replay_us": round(graph_us, 2),
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": round(gbs / peaks["hbm_gbs"], 4),
                         "bytes_per_step": bytes_per_step}}


def _device_inputs(batch, tokens, device, seed, cu=None, with_do=True):
    """Synthetic inputs of the bench distribution generated on the device (large shapes)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    shape = (batch, tokens, H, D)

    def rnd(*s):
        return torch.randn(*s, generator=gen, device=device)

    q = torch.nn.functional.normalize(rnd(*shape), dim=-1).bfloat16()
    k = torch.nn.functional.normalize(rnd(*shape), dim=-1).bfloat16()
    v = rnd(*shape).bfloat16()
    g = torch.nn.functional.logsigmoid(rnd(*shape)).mul_(LOG2E)
    if cu is None:
        pad = (-tokens) % CHUNK
        if pad:
            raise ValueError("dense bench shapes hold whole chunks")
        g = g.view(batch, tokens // CHUNK, CHUNK, H, D).cumsum_(2).view(shape)
    else:   # chunk-local prefix sums restarting at every sequence start
        out = torch.empty_like(g)
        bounds = cu.tolist()
        for a, b in zip(bounds[:-1], bounds[1:]):
            n = b - a
            full = n // CHUNK * CHUNK
            if full:
                out[0, a:a + full] = g[0, a:a + full].view(full // CHUNK, CHUNK, H, D).cumsum(1).view(full, H, D)
            if n > full:
                out[0, a + full:b] = g[0, a + full:b].cumsum(0)
        g = out
    beta = torch.sigmoid(rnd(batch, tokens, H))
    d = {"q": q, "k": k, "v": v, "g": g.contiguous(), "beta": beta}
    if with_do:
        d["do"] = rnd(*shape).bfloat16()
    return d


def bench_other_configs(kda_b200, _cabi, device, iters=5):
    """The two other GPU workloads of the spec, timed with CUDA events (not the headline metric):
    config 2 = 64 packed sequences of 128..8192 tokens with initial states, forward + backward;
    config 4 = one sequence of 1,048,576 tokens, forward."""
    out = {}

    def timed(fn, n):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        _cabi.read_stage_timing(reset=True)
        _cabi.stage_timing(True)
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        z.record()
        torch.cuda.synchronize()
        stages = _cabi.read_stage_timing(reset=True)
        _cabi.stage_timing(False)
        return a.elapsed_time(z) / n, {k: round(v[1] / max(v[0], 1), 4) for k, v in stages.items()}

    # ---- config 2
    gen = torch.Generator().manual_seed(77)
    lengths = torch.randint(128, 8193, (64,), generator=gen)
    cu_host = torch.cat((torch.zeros(1, dtype=torch.int64), lengths.cumsum(0))).to(torch.int32)
    total = int(cu_host[-1])
    cu = cu_host.to(device)
    d = _device_inputs(1, total, device, 78, cu=cu_host)
    h0 = 0.02 * torch.randn(64, H, D, D, device=device)

    def ragged_step():
        leaves = [d[n].detach().requires_grad_() for n in ("q", "k", "v", "g", "beta")]
        h = h0.detach().requires_grad_()
        o, s = kda_b200.chunk_kda(*leaves, h, cu_seqlens=cu, output_final_state=True)
        return torch.autograd.grad((o, s), leaves + [h], (d["do"], torch.ones_like(s)))

    ms, stages = timed(ragged_step, iters)
    out["config2_ragged_fwd_bwd"] = {
        "workload": f"64 packed sequences, 128..8192 tokens each ({total} tokens), H{H}, initial and "
                    "final states with gradients",
        "ms_per_step": round(ms, 3), "tokens_per_s": round(total / (ms * 1e-3), 1),
        "ms_per_kernel_launch": stages}
    del d, h0
    torch.cuda.empty_cache()

    # ---- config 4
    tokens = 1 << 20
    d = _device_inputs(1, tokens, device, 79, with_do=False)

    def long_forward():
        with torch.no_grad():
            return kda_b200.chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], output_final_state=True)

    ms, stages = timed(long_forward, 3)
    out["config4_long_forward"] = {
        "workload": f"one sequence of {tokens} tokens, H{H}, forward with final state",
        "ms_per_step": round(ms, 3), "tokens_per_s": round(tokens / (ms * 1e-3), 1),
        "ms_per_kernel_launch": stages}
    del d
    torch.cuda.empty_cache()
    return out


def bench_preops(device, peaks, batch=8, tokens=4096, iters=20):
    """The bandwidth-bound pre-ops at the config-1 shapes: achieved HBM GB/s of each kernel
    (algorithmic bytes: what its interface must read + write) with CUDA events."""
    ops = torch.ops.kda_b200
    gen = torch.Generator().manual_seed(9)
    n = batch * tokens * H * D
    raw = torch.randn(batch, tokens, H, D, generator=gen).bfloat16().to(device)
    a_log = torch.randn(H, generator=gen).to(device) * 0.1
    dt_bias = torch.randn(H, D, generator=gen).to(device) * 0.1
    dcum = torch.randn(batch, tokens, H, D, generator=gen).to(device)
    x = torch.randn(batch, tokens, H, D, generator=gen).bfloat16().to(device)
    dy = torch.randn(batch, tokens, H, D, generator=gen).bfloat16().to(device)
    y, rstd = ops.kda_l2norm_fwd(x, 1e-6)
    xc = x.view(batch, tokens, H * D)
    dyc = dy.view(batch, tokens, H * D)
    w = (torch.randn(H * D, 4, generator=gen) * 0.5).bfloat16().to(device)
    norm_w = (1 + 0.1 * torch.randn(D, generator=gen)).to(device)
    cases = {
        "gate_cumsum_fwd": (lambda: ops.kda_bounded_gate_fwd_dense(raw, a_log, dt_bias, CHUNK, -5.0), 6),
        "gate_cumsum_bwd": (lambda: ops.kda_bounded_gate_bwd(raw, a_log, dt_bias, dcum, None, None,
                                                             CHUNK, -5.0), 8),
        "l2norm_fwd": (lambda: ops.kda_l2norm_fwd(x, 1e-6), 4),
        "l2norm_bwd": (lambda: ops.kda_l2norm_bwd(y, rstd, dy), 6),
        "short_conv_fwd": (lambda: ops.short_conv_fwd(xc, w, activation="silu"), 4),
        "short_conv_bwd": (lambda: ops.short_conv_bwd(xc, w, dyc, activation="silu"), 6),
        "output_gate_fwd": (lambda: ops.kda_output_gate_fwd(x, raw, norm_w, 1e-5), 6),
        "output_gate_bwd": (lambda: ops.kda_output_gate_bwd(x, raw, norm_w, dy, 1e-5), 10),
    }
    out = {}
    for name, (fn, bytes_per_elem) in cases.items():
        for _ in range(3):
            fn()
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(iters):
            fn()
        z.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(z) * 1e3 / iters
        gbs = n * bytes_per_elem / (us * 1e-6) / 1e9
        out[name] = {"us": round(us, 1), "bytes_per_elem": bytes_per_elem, "achieved_gbs": round(gbs, 1),
                     "frac": round(gbs / peaks["hbm_gbs"], 4)}
    return out


CPU_SAMPLE = "chunk_kda fwd+bwd, B=1 T=1024 H=32 K=V=128, fp32, eager PyTorch on the host cores"


def cpu_sample_step(threads):
    """One bounded CPU sample of the path: B=1 T=1024 H=32 K=V=128 fp32 forward + backward, by the
    reference's own ``chunk_kda(impl="reference")`` when oracle/_ref holds it, else by the oracle
    port.  Returns (tokens, seconds, kind)."""
    from oracle import build_ref
    from oracle import kda_oracle as orc

    torch.set_num_threads(threads)
    inp = orc.make_inputs(1, 1024, H, D, D, seed=7)
    gen = torch.Generator().manual_seed(3)
    do = torch.randn(inp["v"].shape, generator=gen)
    reference_chunk_kda = build_ref.load_reference_chunk_kda()
    t0 = time.perf_counter()
    if reference_chunk_kda is not None:
        leaves = [inp[n].clone().requires_grad_() for n in ("q", "k", "v", "cum_gate", "beta")]
        o, _ = reference_chunk_kda(*leaves, impl="reference")
        torch.autograd.grad(o, leaves, do)
        kind = "reference"
    else:
        orc.chunk_kda_grads_ref(inp["q"], inp["k"], inp["v"], inp["cum_gate"], inp["beta"], do,
                                dtype=torch.float32)
        kind = "port"
    return 1024, time.perf_counter() - t0, kind


def cpu_baseline(bounded=True):
    """One warm-up, then the best of three samples."""
    threads = os.cpu_count() or 1
    cpu_sample_step(threads)
    best = min((cpu_sample_step(threads) for _ in range(3)), key=lambda r: r[1])
    tokens, secs, kind = best
    return {"value": round(tokens / secs, 2), "unit": "tokens/s", "cores": threads, "kind": kind,
            "sample": CPU_SAMPLE + ("" if kind == "reference" else " (oracle port)")
                      + "; 1 warm-up, best of 3"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    kind = "port"
    for _ in range(max(args.warmup, 1)):
        cpu_sample_step(threads)
    total_tokens, total_s = 0, 0.0
    for _ in range(args.steps):
        n, s, kind = cpu_sample_step(threads)
        total_tokens += n
        total_s += s
    value = total_tokens / total_s
    what = ("the reference's chunk_kda(impl=\"reference\") from oracle/_ref" if kind == "reference"
            else "oracle port")
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 2), "unit": "tokens/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(1e3 * total_s / args.steps, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "config1 shape, bounded CPU sample per step: chunk_kda fwd+bwd "
                               f"B=1 T=1024 H={H} K=V={D} chunk={CHUNK} (fp32, host cores)"},
        "cpu_baseline": {"value": round(value, 2), "unit": "tokens/s", "cores": threads,
                         "kind": kind, "sample": f"{what}, B=1 T=1024 H=32 per step"},
        "e2e": {"value": round(value, 2), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--small", action="store_true", help="B=2 T=4096 (for profiler captures)")
    ap.add_argument("--skip-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--skip-e2e", action="store_true", help="skip the host-buffer leg")
    ap.add_argument("--skip-decode", action="store_true", help="skip the decode-step measurement")
    ap.add_argument("--skip-splits", action="store_true",
                    help="skip the strong-scaling and context-parallel legs")
    ap.add_argument("--other-configs", action="store_true",
                    help="also time the packed (config 2) and 1M-token (config 4) workloads")
    ap.add_argument("--cp-only", action="store_true",
                    help="run only the long-sequence forward leg (for profiler captures)")
    ap.add_argument("--cp-tokens", type=int, default=1 << 20,
                    help="tokens of the long-sequence forward leg")
    ap.add_argument("--preops-only", action="store_true",
                    help="measure only the gate / l2norm / short-conv pre-ops (for profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback of the fused path)")
    if args.cp_only:
        import kda_b200
        from kda_b200 import _cabi

        torch.cuda.set_device(0)
        dev0 = torch.device("cuda", 0)
        print(json.dumps({"cp": bench_cp(kda_b200, _cabi, dev0, 0, 1, torch.cuda.synchronize,
                                         tokens=args.cp_tokens)}), flush=True)
        return
    if args.preops_only:
        import kda_b200  # noqa: F401  (registers the operators)
        torch.cuda.set_device(0)
        print(json.dumps({"preops": bench_preops(torch.device("cuda", 0), load_peaks(), iters=3)}), flush=True)
        return
    run_ours(args)


if __name__ == "__main__":
    main()
