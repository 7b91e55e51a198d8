#!/usr/bin/env python
"""Benchmark of the EggRoll population hot path on B200.

Workload (N = 1): the perturbed-linear microbenchmark — per-member input x of
shape [n_pop = 8192, Bm = 16, K = 1024] and W [1024, 1024], fp32 N(0,1), rank-16
factors from the counter RNG (seed key below), one LIF step, spikes out.  A
"step" is one pass of hses_perturbed_linear over that batch.  With N > 1 every
rank runs the same per-GPU batch on its own slice of a population of N*8192
members (weak scaling, no data-path collective: the path emits spikes only).

Metric: member-evaluations per second = n_pop * Bm * T (T = 1) per second.

The same JSON line carries two more blocks, measured after the headline:
  population_step  one full ES step of the spiking MLP 784-128-128-128-10 at 65 536 members of one
                   sample, T = 8, rank 64 (ranks 96 and 128 too on one GPU): encode -> perturbed
                   forward -> fitness -> all-gather -> z-score -> sharded update -> one gradient
                   sum -> AdamW, STRONG scaling (the population is split over the N ranks, both
                   exchanges inside the timed region), with a check that every rank ends a step
                   with bit-identical parameters and that they match the single-GPU step;
  streaming        the HBM-bound kernels of the path (encode, LIF scan, attention, WKV-7), each
                   timed alone against the measured copy bandwidth;
  spiking_lm       (one GPU) the token-level spiking transformer at 4096 members x 32 sequences:
                   ms per fitness evaluation of the whole population;
  rwkv_lm          the 12-layer RWKV-7 LM (d_model 768, vocab 50 277, context 256) evaluated by 1024
                   members with rank-1 noise, bf16 products, the population split over the N ranks.

    python bench.py --gpus N --steps K --warmup W            # the CUDA path
    python bench.py --impl reference --gpus N --steps K ...   # CPU restatement of the reference
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "member_evals_per_sec"
UNIT = "member-evals/s"
KEY = 0x3C6EF372FE94F82A          # base key of parameter index 1
SIGMA, RANK, TAU_M, V_TH = 0.02, 16, 20.0, 0.3
N_POP, BM, K_DIM, A_DIM = 8192, 16, 1024, 1024
# dram__bytes_read.sum + dram__bytes_write.sum of one launch divided by its members, from an ncu
# capture of these kernels at n_pop = 2048: constants of that capture, not a measurement of this run
NCU_TRAFFIC_BYTES_PER_MEMBER = {"linear_tc": (192.4e6 + 90.7e6) / 2048, "lowrank_t": (137.9e6 + 79.8e6) / 2048}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed regions run."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(gpu_index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.tmp.flush()
        rows = []
        with open(self.tmp.name) as fh:
            for line in fh:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) == 7:
                    rows.append(parts)
        os.unlink(self.tmp.name)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(r[0]) for r in rows if r[0].replace(".", "").isdigit())
        # "under load": the upper half of the samples (idle gaps between regions pull the rest down)
        load = sm[len(sm) // 2:] if sm else []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        power = [float(r[2]) for r in rows if r[2].replace(".", "").isdigit()]
        return {"sm_mhz": float(np.median(load)) if load else None,
                "sm_max_mhz": float(rows[0][1]) if rows[0][1].replace(".", "").isdigit() else None,
                "power_w_max": max(power) if power else None, "samples": len(rows), "reasons": reasons}


def synth_inputs(rank: int, n_pop: int):
    """Seeded synthetic inputs of the microbenchmark's shapes (seed 1; ranks differ in x)."""
    g = np.random.Generator(np.random.PCG64(1))
    w = g.standard_normal((A_DIM, K_DIM), dtype=np.float32)   # param = Wᵀ, (a, k)
    gx = np.random.Generator(np.random.PCG64(1000 + rank))
    x = gx.standard_normal((n_pop, BM, K_DIM), dtype=np.float32)
    return x, w


def cpu_rate(oracle, x, w, target_seconds: float, first_thread: int = 0):
    """Times the CPU restatement on a bounded sample: whole passes over the first `members`
    members, repeated until about target_seconds have gone by.  Returns (evals/s, description
    of the sample, seconds)."""
    def one_pass(m):
        oracle.perturbed_linear_lif(x[:m], w, SIGMA, RANK, KEY, first_thread=first_thread, tau_m=TAU_M,
                                    v_th=V_TH, acc64=2)
    probe = min(32, x.shape[0])
    one_pass(probe)                       # thread start-up, page faults
    t0 = time.perf_counter()
    one_pass(probe)
    dt = max(time.perf_counter() - t0, 1e-4)
    members = int(min(x.shape[0], max(probe, probe * target_seconds / dt)))
    members -= members % 2
    passes = 0
    t0 = time.perf_counter()
    while True:
        one_pass(members)
        passes += 1
        dt = time.perf_counter() - t0
        if dt >= target_seconds or passes >= 64:
            break
    return members * passes * BM / dt, f"{passes} pass(es) over {members} of {N_POP} members ({members * BM} rows each)", dt


def config_dict(n_gpus: int):
    return {"workload": f"perturbed-linear microbench: x[{N_POP},16,1024] fp32, W[1024,1024], rank 16, sigma 0.02, "
                        "one LIF step (tau_m 20, v_th 0.3), spikes out",
            "n_pop_per_gpu": N_POP, "bm": BM, "k": K_DIM, "a": A_DIM, "rank": RANK, "t_steps": 1,
            "population_total": N_POP * n_gpus,
            "l2_policy": f"inputs ({N_POP * BM * K_DIM * 4 >> 20} MiB) and outputs ({N_POP * BM * A_DIM * 4 >> 20} MiB) "
                         "exceed the 126 MB L2, no flush needed"}


def run_reference(args, rank: int, world: int):
    if rank != 0:
        return
    from oracle import oracle as O
    O.build()
    # every core this process may run on (a launcher such as torchrun pins OMP_NUM_THREADS to 1)
    O.set_num_threads(len(os.sched_getaffinity(0)))
    # a bounded slice of the same workload: enough members for ~2 s of CPU work per step
    x, w = synth_inputs(0, 512)
    rates = []
    sample = ""
    for i in range(args.warmup + args.steps):
        r, sample, secs = cpu_rate(O, x, w, 2.0)
        if i >= args.warmup:
            rates.append((r, secs))
    total_evals = sum(r * s for r, s in rates)
    total_s = sum(s for _, s in rates)
    value = total_evals / total_s
    cores = O.num_threads()
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total_s / max(len(rates), 1),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": config_dict(args.gpus),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": f"per step: {sample}; C restatement of the reference path, OpenMP over "
                                       "members, register-blocked 4x4 SIMD base product (not a cache-blocked "
                                       "library GEMM)"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
            "note": "the reference's Rust/Burn CPU path cannot be built on this box (no Rust toolchain); "
                    "this is the timed CPU restatement"}
    print(json.dumps(line), flush=True)


def run_ours(args, rank: int, local_rank: int, world: int):
    import torch
    import torch.distributed as dist
    from hyperscalees_b200 import core, ops

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ctx = core.get_context(local_rank)
    peaks = measured_peaks()

    x_np, w_np = synth_inputs(rank, N_POP)
    x_host = torch.from_numpy(x_np).pin_memory()
    w_dev = torch.from_numpy(w_np).to(dev)
    x_dev = torch.empty_like(x_host, device=dev)
    x_dev.copy_(x_host)
    out_dev = torch.empty((N_POP * BM, A_DIM), dtype=torch.float32, device=dev)
    out_host = torch.empty((N_POP * BM, A_DIM), dtype=torch.float32).pin_memory()
    first_thread = rank * N_POP

    def step():
        ops.perturbed_linear(x_dev, w_dev, n_pop=N_POP, bm=BM, sigma=SIGMA, rank=RANK, key=KEY,
                             first_thread=first_thread, lif=True, tau_m=TAU_M, v_th=V_TH, out=out_dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, iters):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        barrier()
        return float(ms.item())

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    ctx.profile_enable(False)
    ms_total = timed(step, args.steps)
    launches = sum(v[0] for v in ctx.profile_read().values())

    # per-kernel device time over the same K steps, CUDA events on the launching stream
    ctx.profile_enable(True)
    timed(step, args.steps)
    prof = {k: v for k, v in ctx.profile_read().items() if v[0]}
    ctx.profile_enable(False)

    # end to end through the public call with host buffers: H2D of the inputs, the step, D2H of the
    # spikes, all inside the timed region; the library's host pipeline overlaps the three on streams
    pipe = ops.HostPipeline(N_POP, BM, K_DIM, A_DIM, chunks=8, device=dev, taper=True)

    def e2e_step():
        pipe.run(x_host, w_dev, out_host, first_thread=first_thread, sigma=SIGMA, rank=RANK, key=KEY,
                 lif=True, tau_m=TAU_M, v_th=V_TH)

    if args.kernel_only:
        ms_e2e = float("nan")
    else:
        for _ in range(2):
            e2e_step()
        ms_e2e = timed(e2e_step, args.steps)
    # Secondary figure: the same step with the factors read from a device-resident cache that was
    # generated once outside the timed region (the reference's LoraNoiseCache mode of operation,
    # valid while the epoch bucket does not change).  The headline above regenerates every step.
    cached = None
    if not args.kernel_only:
        t0 = time.perf_counter()
        cache = ops.FactorCache(KEY, 0, 0, RANK, A_DIM, K_DIM, n_pairs=N_POP // 2,
                                first_pair=first_thread // 2, device=dev)
        torch.cuda.synchronize()
        build_ms = (time.perf_counter() - t0) * 1e3

        def cached_step():
            ops.perturbed_linear(x_dev, w_dev, n_pop=N_POP, bm=BM, sigma=SIGMA, rank=RANK, key=KEY,
                                 first_thread=first_thread, lif=True, tau_m=TAU_M, v_th=V_TH, out=out_dev,
                                 cache=cache)

        for _ in range(3):
            cached_step()
        ms_cached = timed(cached_step, args.steps)
        cached = {"value": N_POP * BM * world * args.steps / (ms_cached * 1e-3), "unit": UNIT,
                  "ms_per_step": ms_cached / args.steps, "cache_bytes_per_gpu": int(cache.data.numel() * 4),
                  "cache_build_ms": build_ms,
                  "note": "factors read from a device cache built once outside the timed region"}
        del cache
    # What bounds the dominant kernel: the clean product alone, and the regeneration of the step's
    # factors alone (the kernel regenerates the output-side half inside its epilogue), both timed here
    floors = None
    if rank == 0:
        def clean_step():
            ops.perturbed_linear(x_dev, w_dev, n_pop=N_POP, bm=BM, perturb=False, lif=True, tau_m=TAU_M, v_th=V_TH,
                                 out=out_dev)

        def regen_all():
            ops.FactorCache(KEY, 0, 0, RANK, A_DIM, K_DIM, n_pairs=N_POP // 2, first_pair=first_thread // 2, device=dev)

        for fn in (clean_step, regen_all):
            for _ in range(3):
                fn()
        torch.cuda.synchronize()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        for _ in range(5):
            clean_step()
        e[1].record()
        for _ in range(5):
            regen_all()
        e[2].record()
        torch.cuda.synchronize()
        normals = (N_POP // 2) * (A_DIM + K_DIM) * RANK
        regen_ms = e[1].elapsed_time(e[2]) / 5
        floors = {"clean_product_step_ms": e[0].elapsed_time(e[1]) / 5,
                  "regenerate_all_factors_ms": regen_ms, "normals_per_step": normals,
                  "generator_G_normals_per_s": normals / (regen_ms * 1e-3) / 1e9,
                  "note": "the step without noise (operand split + GEMM + LIF), and one stand-alone pass that "
                          "regenerates every factor of the step bit-exactly (about 146 instructions per normal); the "
                          "step's kernels do both, half of the factors in each of its two launches"}
    if world > 1:
        dist.barrier()
    # ---- the two extra blocks of the line (see the module docstring) ----
    pop_block, stream_block, lm_block, rwkv_block, einsum_block = None, None, None, None, None
    if not args.kernel_only and not args.headline_only:
        del x_dev, out_dev, pipe
        torch.cuda.empty_cache()
        comm = make_comm(ctx, world)
        pop_block = population_step_case(rank, world, dev, ctx, comm, args.pop_members, 1, 64, "auto",
                                         args.steps, args.warmup, check=True, single_gpu_leg=True)
        if world == 1:
            # the factors regenerated in registers in both halves of the step instead of cached
            regen = population_step_case(rank, world, dev, ctx, comm, args.pop_members, 1, 64, "off",
                                         max(2, args.steps // 4), 3, check=False, single_gpu_leg=False)
            pop_block["regenerating"] = {k: regen[k] for k in ("ms_per_step", "member_evals_per_sec", "kernel_ms_per_step")}
            pop_block["rank_sweep"] = {}
            for r in (96, 128):
                blk = population_step_case(rank, world, dev, ctx, comm, args.pop_members, 1, r, "auto",
                                           args.steps, args.warmup, check=False, single_gpu_leg=False)
                pop_block["rank_sweep"][str(r)] = {k: blk[k] for k in ("ms_per_step", "member_evals_per_sec",
                                                                      "kernel_ms_per_step", "device_status")}
            stream_block = streaming_block(dev, ctx, args.steps, args.warmup,
                                           only=("poisson_encode", "lif_scan", "spiking_attention mode 0", "wkv7"))
            lm_block = spiking_lm_block(dev, ctx, 4096, 32, args.steps, args.warmup)
            einsum_block = einsum_pair_block(dev, ctx, args.steps, args.warmup)
        rwkv_block = rwkv_lm_block(rank, world, dev, ctx, comm, 1024, args.steps, args.warmup)
        if comm is not None:
            comm.destroy()
    clocks = sampler.stop() if sampler else None

    evals_per_step = N_POP * BM * world
    value = evals_per_step * args.steps / (ms_total * 1e-3)
    e2e_value = evals_per_step * args.steps / (ms_e2e * 1e-3)

    if rank == 0:
        top = max(prof.items(), key=lambda kv: kv[1][1])
        top_name, (top_n, top_ms) = top
        rows = N_POP * BM
        # algorithmic work of one launch of the dominant kernel:
        #   GEMM 2*rows*K*A plus the rank-r epilogue 2*rows*r*A
        flops = 2.0 * rows * K_DIM * A_DIM + 2.0 * rows * RANK * A_DIM
        per_launch_s = top_ms * 1e-3 / top_n
        achieved = flops / per_launch_s / 1e12
        roofline = {"kernel": top_name, "bound": "tensor", "achieved": achieved,
                    "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
                    "peak_source": f"{peaks['source']} bf16 cuBLAS burst; the kernel executes three fp16 passes per "
                                   "product (hi*hi + hi*lo + lo*hi) for fp32-equivalent results, so the ceiling "
                                   "for algorithmic flops is one third of the peak",
                    "executed_tflops": 3.0 * achieved,
                    "traffic": NCU_TRAFFIC_BYTES_PER_MEMBER.get(top_name, 0) * N_POP or None,
                    "traffic_source": "constant from the committed ncu summary of this kernel (capture at n_pop = 2048), "
                                      "scaled by the members of one launch; not measured in this run",
                    "algorithmic_flops_per_launch": flops,
                    "avg_launch_ms": per_launch_s * 1e3,
                    "floors": floors,
                    "kernel_time_share": {k: round(v[1] / sum(p[1] for p in prof.values()), 4) for k, v in prof.items()}}
        cpu = None
        if world == 1 and not args.kernel_only:
            from oracle import oracle as O
            O.build()
            O.set_num_threads(len(os.sched_getaffinity(0)))
            r, sample, secs = cpu_rate(O, x_np, w_np, 12.0)
            cpu = {"value": r, "unit": UNIT, "cores": O.num_threads(), "kind": "port",
                   "sample": f"{sample}, {secs:.1f} s; C restatement of the reference path, OpenMP over members, "
                             "register-blocked 4x4 SIMD base product (not a cache-blocked library GEMM)"}
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": config_dict(world), "roofline": roofline, "cpu_baseline": cpu,
                "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                        "h2d_bytes_per_step": int(x_host.numel() * 4), "d2h_bytes_per_step": int(out_host.numel() * 4)},
                "gpu_launches": int(launches), "clocks": clocks, "factor_cache": cached,
                "population_step": pop_block, "streaming": stream_block, "spiking_lm": lm_block,
                "rwkv_lm": rwkv_block, "einsum_pair": einsum_block}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def einsum_pair_block(dev, ctx, steps: int, warmup: int, half: int = 6000, r: int = 64, a: int = 256, b: int = 784):
    """The explicit-input paired einsum (the GPU trainer's einsum_pair_fused) at the shape the reference
    quotes its kernel on: M = 256, N = 784, K = half*r = 384 000.  Times the call on 16-byte aligned
    operands (tensor-core kernel) and on the same values shifted by one float (fp32 kernel), and
    compares a sub-block of both outputs with an fp64 product."""
    import torch
    from hyperscalees_b200 import ops
    g = torch.Generator(device=dev).manual_seed(7)
    flat_a = torch.randn(half * r * a + 4, device=dev, generator=g)
    flat_b = torch.randn(half * r * b + 4, device=dev, generator=g)
    scores = torch.randn(2 * half, device=dev, generator=g)
    peaks = measured_peaks()
    nbytes = 4.0 * half * r * (a + b)
    out = {"shape": {"M": a, "N": b, "K": half * r, "half": half, "r": r},
           "reference_figure": "7.2 ms for the reference's own kernel and 8.4-8.9 ms for its cuBLAS TF32 route, both on an RTX 4090 (docs/cuda_oxide_integration_plan.md:283-299)"}
    for name, off in (("tensor_core", 0), ("fp32_kernel", 1)):
        a_t = flat_a[off:off + half * r * a].view(half, r, a)
        b_t = flat_b[off:off + half * r * b].view(half, r, b)
        for _ in range(max(warmup, 3)):
            g_raw, g_ones = ops.einsum_pair(a_t, b_t, scores)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = steps if off == 0 else max(2, steps // 4)
        e0.record()
        for _ in range(n):
            g_raw, g_ones = ops.einsum_pair(a_t, b_t, scores)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        w = (scores[:half] + scores[half:]).double().repeat_interleave(r)
        A = a_t[:, :, :32].double().reshape(-1, 32)
        B = b_t[:, :, b - 48:].double().reshape(-1, 48)
        ref_raw, ref_ones = (A * w[:, None]).T @ B, 2.0 * (A.T @ B)
        err = max(((g_raw[:32, b - 48:].double() - ref_raw).abs().max() / ref_raw.abs().max()).item(),
                  ((g_ones[:32, b - 48:].double() - ref_ones).abs().max() / ref_ones.abs().max()).item())
        out[name] = {"ms": round(ms, 4), "GB_per_s": round(nbytes / (ms * 1e-3) / 1e9, 1),
                     "frac_of_measured_hbm": round(nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 3),
                     "algorithmic_tflops": round(2 * 2.0 * a * b * half * r / (ms * 1e-3) / 1e12, 1),
                     "max_err_over_largest_entry": float(f"{err:.3g}")}
        del a_t, b_t, g_raw, g_ones
    out["device_status"] = int(ctx.device_status())
    del flat_a, flat_b
    torch.cuda.empty_cache()
    return out


POP_DIMS, POP_T = [784, 128, 128, 128, 10], 8


def pop_inputs(n_total: int, bm: int):
    """Seeded synthetic images of MNIST's shape (each pixel 0 with p = 0.8, else U(0,1); seed 0) and labels."""
    g = np.random.Generator(np.random.PCG64(0))
    img = g.random((n_total * bm, 784), dtype=np.float32)
    img[g.random((n_total * bm, 784)) < 0.8] = 0.0
    return img, g.integers(0, 10, n_total * bm).astype(np.int32)


def population_step_case(rank: int, world: int, dev, ctx, comm, n_total: int, bm: int, r: int, cache: str,
                         steps: int, warmup: int, check: bool, single_gpu_leg: bool, exchange: str = "nccl"):
    """One full ES step of the spiking MLP, the population split over the ranks (strong scaling).
    Per step and rank: encode -> forward -> fitness of its members; all-gather of the raw fitness;
    z-score; contraction of its own members' factors; ONE sum of the flat gradient buffer; the same
    AdamW step everywhere.  Both exchanges go through the library's communicator and are inside the
    timed region.  Returns the block for the JSON line (every rank must call; rank 0's is printed)."""
    import torch
    import torch.distributed as dist
    from hyperscalees_b200 import models, noiser, parallel

    lo, hi = parallel.shard_range(n_total, rank, world)
    img, labels = pop_inputs(n_total, bm)
    di = torch.as_tensor(img[lo * bm:hi * bm], device=dev)
    dl = torch.as_tensor(labels[lo * bm:hi * bm], device=dev)
    keys = models.default_base_keys(len(POP_DIMS))

    def make(first, n_local, cache_policy, whole):
        net = models.SnnMlp(POP_DIMS, tau_m=20.0, v_th=0.3, seed=0, device=dev)
        frozen, nz = noiser.init_noiser(net.params(), 0.02, 0.01, 0, False, 0, r, noiser.Solver.adamw(0.01))
        return models.PopulationStep(net, frozen, nz, keys, POP_T, n_local, bm, first_thread=first,
                                     cache=cache_policy, n_total=n_total if whole else None)

    # exchange "peer": the fitness vector travels through the library's peer-memory kernels (stores into
    # every rank's window over NVLink, a bounded wait) instead of the all-gather
    px = parallel.PeerExchange(n_total, ctx) if (exchange == "peer" and world > 1) else None

    def sharded_step(st):
        raw = st.eval(di, dl, [1, 2, 3, 4 + rank])
        full = px.exchange(raw) if px is not None else parallel.allgather_fitness(raw, n_total, comm=comm)
        st.update_sharded(full, comm=comm)
        return full

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def checksum(params):
        # equal bit patterns give equal sums; the sums of all ranks are compared on rank 0
        return [int(p.view(torch.int32).to(torch.int64).sum().item()) for p in params]

    block = {"workload": f"population step: SNN MLP 784-128-128-128-10, n_pop {n_total}, bm {bm}, T {POP_T}, rank {r}, "
                         f"sigma 0.02, AdamW; factor cache {cache}",
             "n_pop": n_total, "rank": r, "scaling": "strong", "n_gpus": world,
             "parallelism": f"population sharded over {world} GPU(s): fitness all-gather, per-shard partial gradients, "
                            "one gradient sum, identical solver step on every rank"}

    # ---- check: one step from fresh parameters on every rank, against the single-GPU step -------------
    if check:
        st = make(lo, hi - lo, cache, False)
        full = sharded_step(st)
        torch.cuda.synchronize()
        sums = checksum(st.params)
        fsum = int(full.view(torch.int32).to(torch.int64).sum().item())
        gathered = [None] * world
        if world > 1:
            dist.all_gather_object(gathered, (sums, fsum))
        else:
            gathered = [(sums, fsum)]
        block["params_bit_identical_on_all_ranks"] = all(gth == gathered[0] for gth in gathered)
        if rank == 0:
            # the same step on this GPU alone: the shards' forwards as separate calls (the encoder's
            # stream is indexed inside a call's batch and seeded per rank), factors regenerated
            # instead of cached, then the replicated update over the whole fitness vector
            ref = make(0, n_total, "off", True)
            raws = []
            for q in range(world):
                qlo, qhi = parallel.shard_range(n_total, q, world)
                part = make(qlo, qhi - qlo, "off", False)
                part.params, part.net.weights, part.net.out_gain = ref.params, ref.params[:-1], ref.params[-1]
                raws.append(part.eval(torch.as_tensor(img[qlo * bm:qhi * bm], device=dev),
                                      torch.as_tensor(labels[qlo * bm:qhi * bm], device=dev), [1, 2, 3, 4 + q]))
                del part
            raw_ref = torch.cat(raws)
            block["fitness_bit_identical_to_single_gpu"] = bool(torch.equal(raw_ref, full))
            ref.update(raw_ref)
            torch.cuda.synchronize()
            rel = max(((a - b).abs().max() / b.abs().max().clamp_min(1e-12)).item()
                      for a, b in zip(st.params, ref.params))
            block["params_max_rel_diff_to_single_gpu"] = rel
            block["params_within_1e-3_of_single_gpu"] = bool(rel <= 1e-3)
            del ref, raws, raw_ref
        del st
        torch.cuda.empty_cache()
        barrier()

    # ---- timed: K steps, both exchanges inside ------------------------------------------------------
    st = make(lo, hi - lo, cache, False)
    for _ in range(max(warmup, 3)):
        sharded_step(st)
    barrier()
    ctx.profile_enable(False)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        sharded_step(st)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    barrier()
    launches = sum(v[0] for v in ctx.profile_read().values())
    # second pass over the same K steps with per-kernel CUDA events (the exchanges included)
    ctx.profile_enable(True)
    for _ in range(steps):
        sharded_step(st)
    torch.cuda.synchronize()
    prof = {k: v for k, v in ctx.profile_read().items() if v[0]}
    ctx.profile_enable(False)
    status = ctx.device_status()
    del st
    torch.cuda.empty_cache()
    ms_step = float(ms.item()) / steps
    evals = n_total * bm * POP_T
    block.update({"ms_per_step": ms_step, "member_evals_per_sec": evals / (ms_step * 1e-3),
                  "gpu_launches_per_step": launches / steps,
                  "kernel_ms_per_step": {k: round(v[1] / steps, 4) for k, v in sorted(prof.items(), key=lambda kv: -kv[1][1])},
                  "collective_ms_per_step": round(sum(v[1] for k, v in prof.items()
                                                      if k in ("allgather_fitness", "allreduce_grads", "fitness_exchange",
                                                               "fitness_wait")) / steps, 4),
                  "fitness_exchange": "peer memory (hses_fitness_exchange)" if px is not None
                  else "all-gather (hses_allgather_fitness)",
                  "device_status": status})
    if px is not None:
        px.destroy()

    # ---- the whole population on rank 0's GPU alone, in the same job: the strong-scaling yardstick --
    if single_gpu_leg and world > 1:
        barrier()
        if rank == 0:
            one = make(0, n_total, cache, True)
            di1, dl1 = torch.as_tensor(img, device=dev), torch.as_tensor(labels, device=dev)

            def one_step():
                one.update(one.eval(di1, dl1, [1, 2, 3, 4]))

            for _ in range(max(warmup, 3)):
                one_step()
            torch.cuda.synchronize()
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record()
            for _ in range(steps):
                one_step()
            f1.record()
            torch.cuda.synchronize()
            ms1 = f0.elapsed_time(f1) / steps
            block["single_gpu_ms_per_step"] = ms1
            block["speedup_over_single_gpu"] = ms1 / ms_step
            del one, di1, dl1
            torch.cuda.empty_cache()
        barrier()
    return block


def make_comm(ctx, world: int):
    """The library's own communicator (hses_comm_* behind the C ABI); its id travels through the
    torch.distributed group that the launcher's environment already describes."""
    if world == 1:
        return None
    from hyperscalees_b200 import parallel
    return parallel.Comm.from_process_group(ctx)


def run_population_step(args, rank: int, local_rank: int, world: int):
    """--workload population_step: the block above alone, for one rank of the factors."""
    import torch
    import torch.distributed as dist
    from hyperscalees_b200 import core

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ctx = core.get_context(local_rank)
    comm = make_comm(ctx, world)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    block = population_step_case(rank, world, dev, ctx, comm, args.n_pop, args.bm, args.rank, args.cache,
                                 args.steps, args.warmup, check=not args.kernel_only,
                                 single_gpu_leg=not args.kernel_only, exchange=args.exchange)
    clocks = sampler.stop() if sampler else None
    if rank == 0:
        line = {"metric": METRIC, "value": block["member_evals_per_sec"], "unit": UNIT, "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": block["ms_per_step"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": {"workload": block["workload"]}, "population_step": block,
                "gpu_launches": int(block["gpu_launches_per_step"] * args.steps), "clocks": clocks}
        print(json.dumps(line), flush=True)
    if comm is not None:
        comm.destroy()
    if world > 1:
        dist.destroy_process_group()


def streaming_block(dev, ctx, steps: int, warmup: int, shrink: int = 1, only=None):
    """The HBM-bound kernels around the perturbed linear layer, each timed alone with CUDA events on
    inputs larger than L2; algorithmic bytes / time against the measured copy bandwidth.  `only`
    keeps the cases whose name starts with one of the given prefixes."""
    import torch
    from hyperscalees_b200 import ops

    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.rand(*shape, device=dev, generator=g)
    sh = max(1, shrink)   # divides the leading dimension of every case (reduced cases for ncu captures)
    peaks = measured_peaks()
    out = {}

    def run(name, build):
        if only is not None and not any(name.startswith(p) for p in only):
            return
        built = build()
        fn, nbytes = built[0], built[1]
        fmas = built[2] if len(built) > 2 else None
        for _ in range(max(warmup, 3)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": round(ms, 4), "algorithmic_MB": round(nbytes / 1e6, 1), "GB_per_s": round(gbs, 1),
                     "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 3)}
        if fmas is not None:
            # kernels whose arithmetic, not their bytes, sets the floor: fp32 multiply-adds against the
            # rate of the fp32 pipes (SMs x 128 lanes x the device's SM clock limit)
            props = torch.cuda.get_device_properties(dev)
            khz = getattr(props, "clock_rate", 0) or 1965000   # the device's SM clock limit, kHz
            peak = props.multi_processor_count * 128 * khz * 1e3
            out[name]["algorithmic_GFMA"] = round(fmas / 1e9, 2)
            out[name]["frac_of_fp32_fma_peak"] = round(fmas / (ms * 1e-3) / peak, 3)
        del fn
        torch.cuda.empty_cache()

    def poisson():
        probs = rnd(131072 // sh, 784)
        enc_out = torch.empty(8, 131072 // sh, 784, device=dev)
        return (lambda: ops.poisson_encode(probs, 8, (1, 2, 3, 4), out=enc_out)), probs.numel() * 4 + enc_out.numel() * 4

    def lif():
        cur = rnd(8, 131072 // sh, 128)
        v0 = torch.zeros(131072 // sh, 128, device=dev)
        lif_out = torch.empty_like(cur)
        return (lambda: ops.lif_scan(cur, 2.0, 1.0, v=v0, reset_mode=ops.RESET_SUBTRACT, out=lif_out)), \
            2 * cur.numel() * 4 + 2 * v0.numel() * 4

    def attention(mode):
        def build():
            q, k, v = rnd(32768 // sh, 64, 64), rnd(32768 // sh, 64, 64), rnd(32768 // sh, 64, 64)
            # per head and sequence: scores 64 x 64 x 16 and the weighted sum 64 x 64 x 16
            fm = (32768 // sh) * 4 * 2 * 64 * 64 * 16
            return (lambda: ops.spiking_attention(q, k, v, 4, mode=mode)), 4 * q.numel() * 4, fm
        return build

    def wkv():
        wk = [rnd(256 // sh, 256, 12, 64) * 0.5 for _ in range(6)]
        wk[1] = 0.9 + 0.1 * wk[1]
        state = torch.zeros(256 // sh, 12, 64, 64, device=dev)
        # per token and head: decay, (S a) b^T, v k^T on the 64 x 64 state, S a and the readout S r
        fm = (256 // sh) * 256 * 12 * 5 * 64 * 64
        return (lambda: ops.wkv7(*wk, state)), 7 * wk[0].numel() * 4 + 2 * state.numel() * 4, fm

    def norm(kind):
        def build():
            xn = rnd(262144 // sh, 768)
            wn, bn = torch.ones(768, device=dev), torch.zeros(768, device=dev)
            fn = {"layer_norm": lambda: ops.layer_norm(xn, wn, bn), "group_norm": lambda: ops.group_norm(xn, 12, wn, bn),
                  "relu_square": lambda: ops.relu_square(xn), "rate_encode": lambda: ops.rate_encode(xn, 4.0)}[kind]
            return fn, 2 * xn.numel() * 4
        return build

    def solver():
        par, grd = rnd((1 << 26) // sh), rnd((1 << 26) // sh)
        m1, m2 = torch.zeros_like(par), torch.zeros_like(par)
        return (lambda: ops.solver_step(ops.ADAMW, 1, par, grd, m1, m2, weight_decay=0.01)), 7 * par.numel() * 4

    def prng():
        noise = torch.empty((1 << 28) // sh, device=dev)
        return (lambda: ops.prng_normal_half(noise.numel() // 128, 0.0, 1.0, (1, 2, 3, 4), out=noise)), noise.numel() * 4

    run(f"poisson_encode [{131072 // sh}x784] -> T=8", poisson)
    run(f"lif_scan T=8 [{131072 // sh}x128]", lif)
    run(f"spiking_attention mode 0 [{32768 // sh} seq x 64 tok x 4 heads x 16]", attention(0))
    run("spiking_attention mode 2 (relaxation + softmax)", attention(2))
    run(f"wkv7 [{256 // sh} seq x 256 tok x 12 heads x 64]", wkv)
    run(f"layer_norm [{262144 // sh}x768]", norm("layer_norm"))
    run(f"group_norm 12 groups [{262144 // sh}x768]", norm("group_norm"))
    run(f"relu_square [{262144 // sh}x768]", norm("relu_square"))
    run(f"rate_encode [{262144 // sh}x768]", norm("rate_encode"))
    run(f"solver_step AdamW [{(1 << 26) // sh} params]", solver)
    run(f"prng_normal_half [{(1 << 28) // sh} normals]", prng)
    return {"peak": {"hbm_gbs": peaks["hbm_gbs"], "source": peaks["source"]}, "kernels": out,
            "note": "each kernel timed alone, inputs larger than L2; GB/s = algorithmic bytes / CUDA-event time"}


def run_streaming_kernels(args, local_rank: int):
    """--workload streaming_kernels: every streaming kernel of the path, one GPU."""
    import torch
    from hyperscalees_b200 import core

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    ctx = core.get_context(local_rank)
    sampler = ClockSampler(local_rank)
    ctx.profile_enable(False)
    blk = streaming_block(dev, ctx, args.steps, args.warmup, args.shrink)
    launches = sum(v[0] for v in ctx.profile_read().values())
    clocks = sampler.stop()
    print(json.dumps({"metric": "achieved HBM bandwidth of the streaming kernels", "unit": "GB/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": max(args.warmup, 3), "higher_is_better": True,
                      "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "streaming kernels, each timed alone; inputs larger than L2"},
                      "peak": blk["peak"], "kernels": blk["kernels"],
                      "gpu_launches": int(launches), "clocks": clocks,
                      "device_status": ctx.device_status()}), flush=True)


def spiking_lm_block(dev, ctx, n_pop: int, seqs: int, steps: int, warmup: int, chunk_members: int = 1024):
    """BASELINE's token-level spiking transformer: d_model 64, 4 heads, 2 blocks, MLP ratio 4, vocab 256,
    sequences of 64 uniform token ids, Q/K/V as LIF rates over T = 4, causal spike-product attention,
    rank-8 noise on every matrix, `seqs` sequences per member; one step = the next-token
    log-likelihood fitness of every member.  member-evals/s = n_pop * seqs * T per second."""
    import torch
    from hyperscalees_b200 import models
    from hyperscalees_b200.spiking_lm import LmNoise, SpikingLM

    vocab, L, d, H, blocks, T, rank = 256, 64, 64, 4, 2, 4, 8
    model = SpikingLM(vocab, L, d, H, blocks, mlp_ratio=4, T=T, device=dev, seed=2)
    g = torch.Generator(device=dev).manual_seed(2)
    ids = torch.randint(0, vocab, (n_pop, seqs, L), device=dev, generator=g, dtype=torch.int32)
    noise = LmNoise(0.02, rank, models.default_base_keys(len(model.params())), epoch=0, first_thread=0)
    for _ in range(max(min(warmup, 3), 2)):
        fit = model.fitness(ids, noise, chunk_members=chunk_members)
    torch.cuda.synchronize()
    steps = max(2, min(steps, 5))
    ctx.profile_enable(False)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fit = model.fitness(ids, noise, chunk_members=chunk_members)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    launches = sum(v[0] for v in ctx.profile_read().values()) / steps
    ctx.profile_enable(True)
    model.fitness(ids, noise, chunk_members=chunk_members)
    torch.cuda.synchronize()
    prof = {k: v for k, v in ctx.profile_read().items() if v[0]}
    ctx.profile_enable(False)
    return {"workload": f"token-level spiking transformer: {n_pop} members x {seqs} sequences x {L} tokens, vocab {vocab}, "
                        f"d_model {d}, {H} heads, {blocks} blocks, MLP ratio 4, T {T}, rank {rank}, sigma 0.02, "
                        f"chunks of {chunk_members} members",
            "ms_per_step": ms, "member_evals_per_sec": n_pop * seqs * T / (ms * 1e-3),
            "tokens_per_sec": n_pop * seqs * L / (ms * 1e-3), "gpu_launches_per_step": launches,
            "kernel_ms_per_step": {k: round(v[1], 4) for k, v in sorted(prof.items(), key=lambda kv: -kv[1][1])},
            "fitness_finite": bool(torch.isfinite(fit).all().item()), "fitness_mean": float(fit.mean().item()),
            "device_status": ctx.device_status()}


def run_spiking_lm(args, local_rank: int):
    """--workload spiking_lm: the block above alone, one GPU."""
    import torch
    from hyperscalees_b200 import core

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    ctx = core.get_context(local_rank)
    sampler = ClockSampler(local_rank)
    blk = spiking_lm_block(dev, ctx, args.n_pop, args.bm if args.bm > 1 else 32, args.steps, args.warmup, args.chunk)
    print(json.dumps({"metric": METRIC, "value": blk["member_evals_per_sec"], "unit": UNIT, "n_gpus": 1,
                      "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": blk["ms_per_step"],
                      "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": blk["workload"]}, "spiking_lm": blk, "clocks": sampler.stop()}), flush=True)


def rwkv_lm_block(rank: int, world: int, dev, ctx, comm, n_pop: int, steps: int, warmup: int,
                  chunk_members: int = 1024):
    """BASELINE's RWKV-style LM: 12 layers, d_model 768, vocab 50 277, context 256, bf16 weights
    N(0, 0.02) with fp32 state and accumulation, rank-1 noise on every block matrix, one sequence of
    uniform token ids per member; one step = the mean next-token log-likelihood of every member,
    the population split over the ranks (strong scaling) and the fitness vector all-gathered."""
    import torch
    import torch.distributed as dist
    from hyperscalees_b200 import parallel
    from hyperscalees_b200.rwkv_lm import LmNoise, RwkvLM

    n_layer, d, vocab, T = 12, 768, 50277, 256
    model = RwkvLM(n_layer, d, vocab, head_size=64, device=dev, seed=4)
    lo, hi = parallel.shard_range(n_pop, rank, world)
    g = torch.Generator(device="cpu").manual_seed(4)
    ids = torch.randint(0, vocab, (n_pop, T), generator=g, dtype=torch.int32)[lo:hi].to(dev)
    noise = LmNoise(0.02, 1, first_thread=lo)

    def step():
        raw = model.fitness(ids, noise, chunk_members=chunk_members)
        return parallel.allgather_fitness(raw, n_pop, comm=comm)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(2):
        fit = step()
    barrier()
    steps = max(2, min(steps, 3))
    ctx.profile_enable(False)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fit = step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    barrier()
    launches = sum(v[0] for v in ctx.profile_read().values()) / steps
    ctx.profile_enable(True)
    step()
    torch.cuda.synchronize()
    prof = {k: v for k, v in ctx.profile_read().items() if v[0]}
    ctx.profile_enable(False)
    ms = float(ms.item())
    # products of one step: 2 * rows * (sum of the block matrices' sizes * layers + head)
    per_layer = 4 * d * d + 2 * 4 * d * d + 2 * d * (64 + 32 + 64 + 128)
    flops = 2.0 * n_pop * T * (n_layer * per_layer + d * vocab)
    peaks = measured_peaks()
    blk = {"workload": f"RWKV-7 LM: {n_layer} layers, d_model {d}, vocab {vocab}, context {T}, {n_pop} members x 1 sequence, "
                       f"bf16 products with fp32 accumulation, rank-1 noise, sigma 0.02; chunks of {chunk_members} members",
           "n_gpus": world, "scaling": "strong", "ms_per_step": ms, "member_evals_per_sec": n_pop / (ms * 1e-3),
           "tokens_per_sec": n_pop * T / (ms * 1e-3), "product_tflops": flops / (ms * 1e-3) / 1e12,
           "frac_of_measured_bf16_peak": flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"],
           "gpu_launches_per_step": launches,
           "kernel_ms_per_step": {k: round(v[1], 3) for k, v in sorted(prof.items(), key=lambda kv: -kv[1][1])},
           "fitness_finite": bool(torch.isfinite(fit).all().item()), "fitness_mean": float(fit.mean().item()),
           "device_status": ctx.device_status()}
    del model
    torch.cuda.empty_cache()
    return blk


def run_rwkv_lm(args, rank: int, local_rank: int, world: int):
    """--workload rwkv_lm: the block above alone."""
    import torch
    import torch.distributed as dist
    from hyperscalees_b200 import core

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ctx = core.get_context(local_rank)
    comm = make_comm(ctx, world)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    blk = rwkv_lm_block(rank, world, dev, ctx, comm, args.n_pop, args.steps, args.warmup, args.chunk)
    if rank == 0:
        print(json.dumps({"metric": METRIC, "value": blk["member_evals_per_sec"], "unit": UNIT, "n_gpus": world,
                          "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": blk["ms_per_step"],
                          "higher_is_better": True, "scaling": "strong", "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": blk["workload"]}, "rwkv_lm": blk, "clocks": sampler.stop()}), flush=True)
    if comm is not None:
        comm.destroy()
    if world > 1:
        dist.destroy_process_group()


def run_snn_transformer(args, local_rank: int):
    """Secondary workload: forward_batched of the SNN-rate transformer (d_model 64, 4 heads, 2 blocks,
    16 tokens of 49 inputs, T = 4 encoding steps) over a chunk of --n-pop members with rank-8 noise;
    reports member-evaluations/s = n_pop * T per second.  One GPU."""
    import torch
    from hyperscalees_b200 import core, models
    from hyperscalees_b200.snn_transformer import SnnTransformer, TrainNoise

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    ctx = core.get_context(local_rank)
    n, T, nt, tin, d, H, blocks, classes, rank = args.n_pop, 4, 16, 49, 64, 4, 2, 10, 8
    model = SnnTransformer(tin, nt, classes, d, H, blocks, device=dev, seed=2)
    g = torch.Generator(device=dev).manual_seed(2)
    x = (torch.rand(T, n, nt * tin, device=dev, generator=g) < 0.2).float()
    dn = lambda *s: torch.randn(*s, device=dev, generator=g) * 0.02
    noise = TrainNoise(sigma=0.02, rank=rank, base_keys=models.default_base_keys(len(model.params())), epoch=0,
                       first_thread=0, pos_emb=dn(n, nt, d), out_gain=dn(n, 1), beta=dn(n, 1))
    if args.cache == "auto":
        noise.caches = model.build_caches(noise, n)   # a chunk's factors are generated once (forward + gradient share them)
    for _ in range(max(args.warmup, 3)):
        model.forward_batched(x, noise)
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    ctx.profile_enable(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        logits = model.forward_batched(x, noise)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    prof = {k: v for k, v in ctx.profile_read().items() if v[0]}
    ctx.profile_enable(False)
    print(json.dumps({"metric": METRIC, "value": n * T / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
                      "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "dtype": "f32",
                      "data": "synthetic",
                      "config": {"workload": f"SNN-rate transformer forward_batched: {n} members, T {T}, {nt} tokens x {tin}, "
                                             f"d_model {d}, {H} heads, {blocks} blocks, rank {rank}, sigma 0.02; factor cache {args.cache}"},
                      "kernel_ms_per_step": {k: round(v[1] / args.steps, 4) for k, v in sorted(prof.items(), key=lambda kv: -kv[1][1])},
                      "gpu_launches": int(sum(v[0] for v in prof.values())), "clocks": sampler.stop(),
                      "finite": bool(torch.isfinite(logits).all().item()), "device_status": ctx.device_status()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="microbench", choices=["microbench", "population_step", "streaming_kernels", "snn_transformer", "spiking_lm", "rwkv_lm", "einsum_pair"],
                    help="microbench: the perturbed-linear layer the metric is quoted on (default); "
                         "population_step: a full ES step of the spiking MLP (secondary figure); "
                         "streaming_kernels: the HBM-bound kernels of the path, each timed alone; "
                         "snn_transformer: forward_batched of the SNN-rate transformer over --n-pop members")
    ap.add_argument("--bm", type=int, default=1, help="population_step: samples per member")
    ap.add_argument("--rank", type=int, default=64, help="population_step: rank of the factors")
    ap.add_argument("--cache", default="off", choices=["off", "auto"],
                    help="population_step: keep the factors of an epoch bucket on the device")
    ap.add_argument("--n-pop", type=int, default=8192,
                    help="microbench: members per GPU (smaller values give the reduced case used for ncu "
                         "captures); population_step: members of the whole population")
    ap.add_argument("--chunk", type=int, default=1024, help="spiking_lm: members evaluated per pass")
    ap.add_argument("--shrink", type=int, default=1,
                    help="streaming_kernels, einsum_pair: divide every case's leading dimension (reduced cases for "
                         "ncu captures)")
    ap.add_argument("--exchange", default="nccl", choices=["nccl", "peer"],
                    help="population_step: how the fitness vector reaches every rank (the library's all-gather, or "
                         "its peer-memory kernels)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end and CPU legs and the extra blocks (profiling runs)")
    ap.add_argument("--headline-only", action="store_true",
                    help="microbench: leave out the population_step and streaming blocks")
    ap.add_argument("--pop-members", type=int, default=65536,
                    help="microbench: population of the population_step block")
    args = ap.parse_args()
    globals()["N_POP"] = args.n_pop
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif args.workload == "population_step":
        run_population_step(args, rank, local_rank, world)
    elif args.workload == "streaming_kernels":
        if rank == 0:
            run_streaming_kernels(args, local_rank)
    elif args.workload == "snn_transformer":
        if rank == 0:
            run_snn_transformer(args, local_rank)
    elif args.workload == "spiking_lm":
        if rank == 0:
            run_spiking_lm(args, local_rank)
    elif args.workload == "rwkv_lm":
        run_rwkv_lm(args, rank, local_rank, world)
    elif args.workload == "einsum_pair":
        if rank == 0:
            import torch
            from hyperscalees_b200 import core
            dev = torch.device("cuda", local_rank)
            torch.cuda.set_device(dev)
            blk = einsum_pair_block(dev, core.get_context(local_rank), args.steps, args.warmup,
                                    half=6000 // max(1, args.shrink))
            print(json.dumps({"workload": "einsum_pair", **blk}), flush=True)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
