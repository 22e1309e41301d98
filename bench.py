"""Benchmark of the Pairformer triangle hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens 3072] [--impl reference]

One "step" = the triangle path of one Pairformer block (tri-mult outgoing,
tri-mult incoming, tri-attention starting node, tri-attention ending node, each
with its residual add) on a synthetic pair tensor z[N,N,128] in bf16 with
random-init N(0, 0.02) weights and a pad mask on the last ~2 % of tokens - the
per-block work of the 48-block trunk at N = 3012 -> 3072 tokens.

Prints ONE JSON line (rank 0): metric = achieved TFLOP/s over the algorithmic
flops of the four ops, ms_per_step = block milliseconds. With N > 1 GPUs the same
complex is sharded over a 1x2 / 2x2 / 2x4 grid (2-D context parallelism, strong
scaling): the value is the whole job's flops over the slowest rank's time.
`--impl reference` times the CPU restatement of the reference's XLA path (the
reference's JAX code cannot run here: JAX is not installed) on a bounded sample.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "pairformer_triangle_block_tflops"
UNIT = "TFLOP/s"


def block_flops(n: int) -> float:
    return 2.0 * (256.0 * n**3 + 196608.0 * n**2) + 2.0 * (512.0 * n**3 + 164864.0 * n**2)


def single_track_flops(n: int, c_s: int = 384, heads: int = 16, c_z: int = 128) -> float:
    """Single track of a block: five c_s x c_s projections, the 128 -> heads pair bias, the token
    attention, and the c_s -> 4 c_s -> c_s transition."""
    return (5 * 2.0 * n * c_s * c_s + 2.0 * n * n * c_z * heads + 4.0 * n * n * c_s + 3 * 2.0 * n * c_s * 4 * c_s)


def make_params(rng: np.random.Generator) -> dict:
    from foldjax_b200.synthetic import block_params

    return block_params(rng)


def measured_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# ----------------------------------------------------------------------- CPU arm
def cpu_block(params, z, mask, dtype="float32"):
    """The oracle's restatement of the reference's XLA path, four ops with residuals."""
    from oracle import triangle_oracle as orc

    z = z + orc.triangle_multiplication(params["tri_mul_out"], z, mask, "outgoing", dtype=dtype)
    z = z + orc.triangle_multiplication(params["tri_mul_in"], z, mask, "incoming", dtype=dtype)
    # attention rows are independent: chunks of rows run on half of the cores, the other half is
    # left to the BLAS threads inside each chunk (one chunk per core oversubscribes and is slower)
    threads = max(1, len(os.sched_getaffinity(0)) // 2)
    z = z + orc.triangle_attention(params["tri_att_start"], z, mask, starting=True, dtype=dtype, threads=threads)
    z = z + orc.triangle_attention(params["tri_att_end"], z, mask, starting=False, dtype=dtype, threads=threads)
    return z


def time_cpu(n: int, reps: int, warmup: int = 0) -> tuple[float, float]:
    """(seconds per block, TFLOP/s) of the CPU restatement at n tokens, fp32, BLAS-threaded."""
    from foldjax_b200.synthetic import pad_mask

    rng = np.random.default_rng(2)
    params = make_params(rng)
    z = rng.standard_normal((1, n, n, 128)).astype(np.float32)
    mask = pad_mask(n, max(1, n // 50))
    for _ in range(warmup):
        cpu_block(params, z, mask)
    t0 = time.perf_counter()
    for _ in range(reps):
        cpu_block(params, z, mask)
    dt = (time.perf_counter() - t0) / reps
    return dt, block_flops(n) / dt / 1e12


def time_cpu_config1() -> dict:
    """BASELINE config 1 in full on the host cores: tri-mult outgoing then incoming, N = 256,
    float32, all-ones mask, seed 0, through the NumPy restatement of the reference's jnp path."""
    from oracle import triangle_oracle as orc

    rng = np.random.default_rng(0)
    n = 256
    params = orc.random_trimul_params(rng)
    x = rng.standard_normal((1, n, n, 128)).astype(np.float32)
    mask = np.ones((1, n, n), np.float32)
    t0 = time.perf_counter()
    orc.triangle_multiplication(params, x, mask, "outgoing", dtype="float32")
    orc.triangle_multiplication(params, x, mask, "incoming", dtype="float32")
    dt = time.perf_counter() - t0
    flops = 2.0 * (256.0 * n**3 + 196608.0 * n**2)
    return {"config": "1: tri-mult out+in N=256 fp32", "seconds": dt, "tflops": flops / dt / 1e12,
            "cores": len(os.sched_getaffinity(0))}


def time_cpu_config3() -> dict:
    """BASELINE config 3 in full on the host cores: one whole Pairformer block, N = 1024 with the
    last 21 tokens padded, through the NumPy restatement (float32 arithmetic)."""
    from oracle import triangle_oracle as orc

    rng = np.random.default_rng(2)
    n = 1024
    params = orc.random_pairformer_params(rng)
    z = rng.standard_normal((1, n, n, 128)).astype(np.float32)
    sv = rng.standard_normal((1, n, 384)).astype(np.float32)
    pair_mask = orc.pad_mask(n, 21)
    mask = np.ones((1, n), np.float32)
    mask[0, n - 21:] = 0.0
    t0 = time.perf_counter()
    orc.pairformer_layer(params, sv, z, mask, pair_mask, dtype="float32")
    dt = time.perf_counter() - t0
    flops = block_flops(n) + 2.0 * n * n * 3 * 128 * 512 + single_track_flops(n)
    return {"config": "3: full Pairformer block N=1024 (21 padded)", "seconds": dt, "tflops": flops / dt / 1e12,
            "cores": len(os.sched_getaffinity(0))}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0))
    n = args.cpu_tokens
    secs, tf = time_cpu(n, reps=max(1, args.steps), warmup=min(1, args.warmup))
    sample = f"one block's four triangle ops at N={n} fp32 (bounded sample of the N={args.tokens} workload)"
    line = {
        "impl": "reference",
        "metric": METRIC, "value": tf, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": secs * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"pairformer-triangle-block N={args.tokens} c_z=128 4x32 heads (cfg 4 per block)",
                   "cpu_sample_tokens": n},
        "cpu_baseline": {"value": tf, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference jnp path unavailable on this box (JAX not installed); NumPy restatement timed instead",
        "cpu_configs_in_full": [time_cpu_config1()] + ([time_cpu_config3()] if args.cpu_config3 else []),
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------- GPU arm
class ClockSampler:
    """nvidia-smi samples of one GPU during the timed region."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def run_gpu(args) -> None:
    import torch
    import torch.distributed as dist

    from foldjax_b200 import _device as dev
    from foldjax_b200 import _lib
    from foldjax_b200.block import triangle_block_forward
    from foldjax_b200.synthetic import pad_mask

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = _lib.load()

    n = args.tokens
    rng = np.random.default_rng(3)
    from foldjax_b200.synthetic import block_params

    # one parameter set per block of the trunk slice (--blocks, default 1 = the headline block)
    trunk = [dev.params_to_device(make_params(rng) if not args.transition else block_params(rng, transition=True))
             for _ in range(args.blocks)]
    params = trunk[0]
    n_pad = args.pad_tokens if args.pad_tokens >= 0 else (n - int(round(n * 3012 / 3072)) if n >= 64 else 0)
    pair_mask = pad_mask(n, n_pad)
    if args.chains:
        # block-diagonal intra-chain mask: a pair survives only inside one chain (whole key tiles masked)
        sizes = [int(v) for v in args.chains.split(",")]
        if sum(sizes) != n:
            raise SystemExit(f"--chains sizes sum to {sum(sizes)}, not to --tokens {n}")
        chain = np.repeat(np.arange(len(sizes)), sizes)
        pair_mask = pair_mask * (chain[:, None] == chain[None, :]).astype(np.float32)[None]
    mask_host = torch.from_numpy(pair_mask).pin_memory()
    mask = mask_host.cuda()
    s_dev = s_host = tok_mask = None
    if args.full_block:
        if world != 1:
            raise SystemExit("--full-block runs on one GPU (the single track is not sharded)")
        # the whole block through the one-call entry: pair track + pair transition + single track
        from foldjax_b200.pairformer import pairformer_forward
        from foldjax_b200.synthetic import pairformer_params

        full = [dev.params_to_device(pairformer_params(rng)) for _ in range(args.blocks)]
        gen = torch.Generator(device="cuda").manual_seed(3)
        z = torch.randn(1, n, n, 128, device="cuda", generator=gen).to(torch.bfloat16)
        s_dev = torch.randn(1, n, 384, device="cuda", generator=gen)
        s_host = s_dev.cpu().pin_memory()
        tok_mask = torch.ones(1, n, device="cuda")
        if n_pad:
            tok_mask[0, n - n_pad:] = 0.0
        def run_block(zz, mm, ss=None):
            return pairformer_forward(full, s_dev if ss is None else ss, zz, tok_mask, mm)[1]
        grid_name = "single GPU, one library call per step"
    elif world == 1:
        gen = torch.Generator(device="cuda").manual_seed(3)
        z = torch.randn(1, n, n, 128, device="cuda", generator=gen).to(torch.bfloat16)
        def run_block(zz, mm):
            for blk in trunk:
                zz = triangle_block_forward(blk, zz, mm)
            return zz
        grid_name = "single GPU"
    else:
        # one complex sharded over an R x C grid: every rank owns one tile of z (2-D
        # context parallelism), the whole [N, N] mask is replicated
        from foldjax_b200 import cp

        ctx = cp.context_parallel()
        n_r, n_c = ctx.grid.tile_shape(n)
        gen = torch.Generator(device="cuda").manual_seed(3 + rank)
        z = torch.randn(n_r, n_c, 128, device="cuda", generator=gen).to(torch.bfloat16)
        mask = mask[0].contiguous()
        mask_host = mask_host[0]
        def run_block(zz, mm):
            for blk in trunk:
                zz = cp.triangle_block_cp(ctx, blk, zz, mm)
            return zz
        run_block(z, mask)  # sizes the exchange workspace (and maps the peers') before anything is timed
        pulls = bool(lib.b200tri_comm_pulls(ctx.comm))
        grid_name = (f"2-D context parallel {ctx.grid.rows}x{ctx.grid.cols}, tiles " +
                     (f"{cp.TRANSPORT}ed through the peers' mapped workspaces by copy engines, {cp.COPY_STREAMS} copy stream(s) "
                      "(NCCL carries tokens only)" if pulls
                      else "exchanged with NCCL point-to-point send/receive"))
    z_host = torch.empty(z.shape, dtype=torch.bfloat16, pin_memory=True)
    z_host.copy_(z)
    out_host = torch.empty_like(z_host).pin_memory()

    def run_e2e():
        if args.full_block:
            zd, sd = z_host.cuda(non_blocking=True), s_host.cuda(non_blocking=True)
            md = mask_host.cuda(non_blocking=True)
            s_new, z_new = pairformer_forward(full, sd, zd, tok_mask, md)
            out_host.copy_(z_new, non_blocking=True)
            s_host.copy_(s_new, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return out_host
        if world == 1 and args.blocks == 1:
            return triangle_block_forward(params, z_host, mask_host, out=out_host)
        zd = z_host.cuda(non_blocking=True)
        md = mask_host.cuda(non_blocking=True)
        out_host.copy_(run_block(zd, md), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return out_host

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing (inputs already in HBM)
    for _ in range(args.warmup):
        run_block(z, mask)
    lib.b200tri_timing_reset()
    lib.b200tri_timing_enable(1)
    launches0 = lib.b200tri_launch_count()
    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        result = run_block(z, mask)
    e1.record()
    barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop() if sampler else None
    launches = int(lib.b200tri_launch_count() - launches0)
    lib.b200tri_timing_enable(0)
    ktimes = _lib.kernel_times()
    if world > 1 and rank == 0 and os.environ.get("B200TRI_BENCH_EXCHANGE_TRACE"):
        # per exchange group of the last step, in order: (whole span, wait for the peers, copies) in ms
        spans = [_lib.kernel_time_list(k) for k in ("cp_exchange", "cp_ready", "cp_copy")]
        per = len(spans[0]) // max(args.steps, 1)
        print("exchange trace:", [tuple(round(v[-per + i], 3) for v in spans if len(v) == len(spans[0]))
                                  for i in range(per)], file=sys.stderr)
    _lib.device_status()
    assert torch.isfinite(result.float()).all(), "non-finite values in the block output"

    # ---- end to end: host buffers in, host buffers out, every step's copies inside the timed
    # region. One call at a time first (what a single complex costs: copy in, block, copy out,
    # nothing to overlap), then the same steps as a stream of complexes through the pipelined
    # entry, which copies step k+1 in and step k-1 out while step k computes.
    e2e_steps = 0 if args.no_e2e else max(1, min(args.steps, 3))
    for _ in range(0 if args.no_e2e else min(args.warmup, 1)):
        run_e2e()
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(e2e_steps):
        run_e2e()
    t1.record()
    barrier()
    e2e_single_ms = max_over_ranks(t0.elapsed_time(t1)) / max(e2e_steps, 1)
    e2e_ms, e2e_mode = e2e_single_ms, "one call per step, copies not overlapped"
    if not args.no_e2e and not args.full_block:
        from foldjax_b200.block import stream_host_blocks

        z_host2 = torch.empty_like(z_host).pin_memory()
        z_host2.copy_(z_host)
        out_host2 = torch.empty_like(z_host).pin_memory()
        pipe_steps = max(args.steps, 2)
        items = [((z_host, z_host2)[k & 1], mask_host) for k in range(pipe_steps)]
        outs = [(out_host, out_host2)[k & 1] for k in range(pipe_steps)]
        stream_host_blocks(run_block, items[:2], outs[:2])  # warm-up: streams, slots, allocator
        barrier()
        t0.record()
        stream_host_blocks(run_block, items, outs)
        t1.record()
        barrier()
        e2e_ms = max_over_ranks(t0.elapsed_time(t1)) / pipe_steps
        e2e_steps = pipe_steps
        e2e_mode = (f"{pipe_steps} steps through stream_host_blocks: the copies of step k+1 (in) and k-1 (out) "
                    "overlap the kernels of step k; fill and drain included")
        assert torch.isfinite(out_host2.float()).all(), "non-finite values in the streamed output"
        del z_host2, out_host2

    # ---- the pair transition that follows the triangle ops in the block (row-local, so
    # every rank runs it on its own tile); reported beside the headline, not inside it
    from foldjax_b200.synthetic import transition_params
    from foldjax_b200.transition import transition_forward

    tparams = dev.params_to_device(transition_params(np.random.default_rng(4)))
    tz, tout = (z if world > 1 else z[0]), torch.empty_like(z if world > 1 else z[0])
    for _ in range(2):
        transition_forward(tparams, tz, residual=tz, out=tout)
    barrier()
    t0.record()
    for _ in range(4):
        transition_forward(tparams, tz, residual=tz, out=tout)
    t1.record()
    barrier()
    transition_ms = max_over_ranks(t0.elapsed_time(t1)) / 4
    del tout

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    ms_step = ms_total / args.steps
    with_transition = args.transition or args.full_block
    flops = args.blocks * (block_flops(n) + (2.0 * n * n * 3 * 128 * 512 if with_transition else 0.0)
                           + (single_track_flops(n) if args.full_block else 0.0))
    peaks, peak_kind = measured_peaks()
    core_ms, core_n = ktimes["triatt_core"]
    core_avg = core_ms / max(core_n, 1)
    # QK^T + PV of the two attention ops of a step, this rank's share (one launch per key tile)
    core_flops_rank = 2.0 * 4.0 * n**3 * 128.0 / world * args.steps * args.blocks
    achieved = core_flops_rank / (core_ms * 1e-3) / 1e12 if core_ms else None
    peak = float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops", 1400.0)))
    exchange_ms, exchange_n = ktimes.pop("cp_exchange", (0.0, 0))  # a span on the exchange stream, not a kernel
    ready_ms = ktimes.pop("cp_ready", (0.0, 0))[0]  # of which: waiting for the peers' "tiles are ready" tokens
    copy_ms = ktimes.pop("cp_copy", (0.0, 0))[0]    # and the pulls plus the "consumed" token round
    shares = {k: round(v[0] / max(sum(t[0] for t in ktimes.values()), 1e-9), 4) for k, v in ktimes.items()}
    cores = len(os.sched_getaffinity(0))
    cpu_secs, cpu_tf = time_cpu(args.cpu_tokens, reps=1) if world == 1 and not args.no_cpu else (None, None)
    line = {
        "metric": METRIC, "value": flops / (ms_step * 1e-3) / 1e12, "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {
            "workload": (f"pairformer-full-block N={n} c_z=128 c_s=384 (cfg 3 at N=1024/21 padded): tri-mult out+in, "
                         "tri-attn start+end, pair transition, single attention with pair bias, single transition"
                         if args.full_block else
                         f"pairformer-triangle-block N={n} c_z=128 4x32 heads (cfg 4 per block): "
                         "tri-mult out+in, tri-attn start+end, residual adds fused"),
            "tokens": n, "pad_tokens": n_pad, "chains": args.chains or None, "flops_per_step": flops, "blocks_per_step": args.blocks,
            "pair_transition_in_step": bool(with_transition), "single_track_in_step": bool(args.full_block),
            "parallelism": grid_name,
            "l2": "inputs larger than L2 (pair tensor %.2f GB)" % (n * n * 128 * 2 / 1e9),
        },
        "clocks": clocks,
        "e2e": None if args.no_e2e else {
                "value": flops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms, "steps": e2e_steps,
                "mode": e2e_mode, "single_call_ms_per_step": e2e_single_ms,
                "single_call_value": flops / (e2e_single_ms * 1e-3) / 1e12,
                "h2d_bytes_per_step": int(world * (z_host.numel() * 2 + mask_host.numel() * 4)
                                          + (s_host.numel() * 4 if args.full_block else 0)),
                "d2h_bytes_per_step": int(world * out_host.numel() * 2 + (s_host.numel() * 4 if args.full_block else 0))},
        "gpu_launches": launches,
        "roofline": {
            "kernel": "att_core_kernel", "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": (achieved / peak) if achieved else None, "peak_kind": f"{peak_kind} sustained bf16",
            # dram read + write bytes per launch measured with ncu's DRAM counters at N = 1024 (this
            # kernel) and N = 3072 (the same load pattern, one-off full-size capture); the traffic is
            # not proportional to N (L2 hit rates change), so it is null at other sizes
            "traffic": {1024: 1.93e9, 3072: 5.55e10}.get(n) if world == 1 else None,
            "avg_launch_ms": core_avg, "launches": core_n,
            "note": "binding resource is the MUFU/ALU softmax path (4*N^3 exps), not the tensor pipe",
        },
        "pair_transition": {
            "ms": transition_ms, "tflops": 2.0 * n * n * 3 * 128 * 512 / (transition_ms * 1e-3) / 1e12,
            "gbs": 3.0 * n * n * 256 / world / (transition_ms * 1e-3) / 1e9,
            "note": "LN + SwiGLU 128->512->128 + residual, one kernel; not part of `value`"},
        "kernel_ms_per_launch": {k: round(v[0] / max(v[1], 1), 4) for k, v in ktimes.items()},
        # rank 0's timed kernels per step against the step: the rest is exchange that the tile compute
        # did not hide, small untimed kernels and launch gaps
        "kernel_ms_per_step": round(sum(v[0] for v in ktimes.values()) / args.steps, 4),
        "non_kernel_ms_per_step": round(ms_step - sum(v[0] for v in ktimes.values()) / args.steps, 4),
        # context-parallel runs: time the send/receive groups spent on the exchange stream per step
        # (transfer time plus waiting for the peers; part of it overlaps the attention core)
        "cp_exchange_ms_per_step": round(exchange_ms / args.steps, 4) if world > 1 else None,
        "cp_ready_wait_ms_per_step": round(ready_ms / args.steps, 4) if world > 1 else None,
        "cp_copy_ms_per_step": round(copy_ms / args.steps, 4) if world > 1 else None,
        "cp_exchange_groups_per_step": exchange_n // max(args.steps, 1) if world > 1 else None,
        "kernel_time_share": shares,
        "cpu_baseline": None if cpu_tf is None else {
            "value": cpu_tf, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"one block's four triangle ops at N={args.cpu_tokens} fp32 via the NumPy restatement "
                      f"({cpu_secs:.1f} s)",
            "configs_in_full": [time_cpu_config1()] + ([time_cpu_config3()] if args.cpu_config3 else [])},
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=3072)
    ap.add_argument("--blocks", type=int, default=1,
                    help="blocks per step, each with its own weights (48 = the trunk of the headline config)")
    ap.add_argument("--transition", action="store_true",
                    help="include the pair transition in every block of the step (and in its flop count)")
    ap.add_argument("--pad-tokens", type=int, default=-1,
                    help="trailing padded tokens in the mask (default: the 3012-of-3072 ratio of the headline config)")
    ap.add_argument("--chains", default="",
                    help="comma-separated chain lengths: adds a block-diagonal intra-chain pair mask "
                         "(the second reading of the N=8192 three-chain case)")
    ap.add_argument("--cpu-tokens", type=int, default=384, help="size of the bounded CPU sample")
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--cpu-config3", action="store_true",
                    help="also time BASELINE config 3 (a whole block at N=1024) in full on the host cores (minutes)")
    ap.add_argument("--full-block", action="store_true",
                    help="one step = the WHOLE Pairformer block through the one-call entry: pair track with the pair "
                         "transition, and the float32 single track (BASELINE config 3 with --tokens 1024 --pad-tokens 21)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
