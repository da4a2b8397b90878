"""Benchmark of the splat hot path: gaussian x pixel evaluations per second, forward +
backward, on the batched training shape (B=16, N=8192, 256x256, C=3, fp32) per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl reference]

For N > 1 launch under torchrun (one rank per GPU); the batch is sharded, every rank
renders its own B=16 block (weak scaling), there is no data-path collective.

One JSON line is printed by rank 0.  ``value`` is measured with inputs resident on the
device; ``e2e`` is the same metric through the public API from pinned host buffers with
host<->device copies inside the timed region.  ``--impl reference`` times the CPU
restatement of the reference's chunked torch path on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# dram__bytes_read.sum + dram__bytes_write.sum per launch, from the ncu captures
# summarised under profiles/ (workload -> kernel -> bytes)
NCU_DRAM_BYTES_PER_LAUNCH = {
    # profiles/splat_kernels_cfg2_dram.md
    "cfg2": {"forward": 18.93e6 + 8.23e6, "backward": 31.38e6 + 8.05e6},
    "cfg2_sep": {"forward": 6.90e6 + 8.56e6, "backward": 26.76e6 + 7.62e6},
    # profiles/splat_kernels_cfg2_small_ncu_full.md
    "cfg2_small": {"forward": 3.46e6 + 0.01e6, "backward": 7.03e6},
    # profiles/splat_sep_kernels_cfg2_small_ncu_full.md
    "cfg2_small_sep": {"forward": 0.98e6 + 0.02e6, "backward": 5.98e6},
}

METRIC = "gaussian_pixel_evals_per_s_fwd_bwd"
UNIT = "evals/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg2", choices=["cfg0", "cfg2", "cfg2_small", "cfg3", "cfg4_b8", "cfg4", "narrow", "narrow64k"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-culling", action="store_true", help="switch the lossless culling off (for comparison)")
    ap.add_argument("--backward-sort", choices=["auto", "on", "off"], default="auto",
                    help="spatial processing order of the backward's gaussians (results are the same bits)")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="budget of the CPU baseline leg")
    return ap.parse_args()


# ---------------------------------------------------------------------------
# clocks during the timed region
# ---------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi (SM clock, power, throttle reasons) of one GPU every 50 ms."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        self.thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), line.strip()))

    def stop(self, t0=None, t1=None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], None, [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ts, line in self.rows:
            if t0 is not None and not (t0 <= ts <= t1 + 0.25):
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax,
                "power_w_max": max(power) if power else None, "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------
# CPU baseline (restatement of the reference's chunked torch path)
# ---------------------------------------------------------------------------
def cpu_step_fn(cfg, n_sample, threads):
    """Returns (step callable, evals per step, description).  The sample keeps the full
    batch and the full image and takes the first n_sample gaussians (a multiple of the
    reference's chunk of 32): the reference's loop runs N/32 identical iterations over
    [B,32,H,W] blocks, so the sample has the working set and the evals/s of the whole
    workload."""
    import torch

    from igs_b200 import workloads
    from oracle import chunked_port as cp

    torch.set_num_threads(threads)
    d = workloads.draw(cfg, N=n_sample, device="cpu")

    def step():
        out, grads = cp.render_fwd_bwd(d["positions"], d["colors"], d["scales"], d["rotations"], d["alphas"], d["x"],
                                       d["y"], lambda o: 2 * (o - d["target"]) / o.numel())
        return grads

    return (step, cfg.B * n_sample * cfg.H * cfg.W,
            f"full batch B={cfg.B}, first {n_sample} of {cfg.N} gaussians, full {cfg.H}x{cfg.W} image")


def calibrate_cpu_sample(cfg, threads, target_s):
    """Gaussians per CPU step so that one step takes about target_s seconds."""
    step, ev, _ = cpu_step_fn(cfg, 32, threads)
    step()
    t0 = time.perf_counter()
    step()
    dt = max(time.perf_counter() - t0, 1e-4)
    n = int(32 * target_s / dt) // 32 * 32
    return max(32, min(cfg.N, n))


def run_cpu_baseline(cfg, seconds):
    threads = os.cpu_count() or 1
    n = calibrate_cpu_sample(cfg, threads, max(seconds / 4.0, 0.5))
    step, ev, sample = cpu_step_fn(cfg, n, threads)
    step()  # warm-up
    times = []
    t_end = time.perf_counter() + seconds * 0.6
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 10):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    res = {"value": ev / med, "unit": UNIT, "cores": threads, "kind": "port",
           "sample": f"{sample}; median of {len(times)} steps of {med:.2f} s; torch restatement of the reference's "
                     "chunked path (oracle/chunked_port.py)"}
    # the fused C oracle on the same sample, for context (a different cost structure)
    try:
        import numpy as np

        from igs_b200 import workloads
        from oracle import splat_oracle as so

        d = {k: v.numpy() for k, v in workloads.draw(cfg, N=n, device="cpu").items()}
        t0 = time.perf_counter()
        so.render_with_grads(d["positions"], d["colors"], d["scales"], d["rotations"], d["alphas"], d["x"][:, 0],
                             d["y"][:, 0], lambda o: 2 * (o - d["target"]) / o.size, dtype=np.float32)
        res["c_oracle_value"] = ev / (time.perf_counter() - t0)
        res["c_oracle_threads"] = so.num_threads()
    except Exception as exc:  # noqa: BLE001 - context only
        res["c_oracle_value"] = None
        res["c_oracle_error"] = str(exc)[:200]
    return res


def run_reference_arm(args):
    """`--impl reference`: the reference's CPU path (its torch restatement) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from igs_b200 import workloads

    cfg = workloads.CONFIGS[args.workload]
    threads = os.cpu_count() or 1
    # size each step to ~1.5 s so that steps + warm-ups stay within a few minutes
    budget = 150.0 / max(args.steps + args.warmup, 1)
    n = calibrate_cpu_sample(cfg, threads, min(1.5, budget))
    step, ev, sample = cpu_step_fn(cfg, n, threads)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = ev * args.steps / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"each step: {sample}; torch restatement of the reference's chunked path "
                                   "(oracle/chunked_port.py; the reference is Python and does not travel)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def workload_config(cfg, n_gpus, by_gaussians=False):
    if by_gaussians:
        return {"workload": f"{cfg.name}: B={cfg.B}, N={cfg.N} split over the GPUs, {cfg.H}x{cfg.W}, C={cfg.C}, fp32, "
                            f"MSE loss, fwd+bwd", "B_per_gpu": cfg.B, "global_batch": cfg.B, "N": cfg.N, "H": cfg.H,
                "W": cfg.W, "C": cfg.C,
                "parallelism": f"gaussian ranges x{n_gpus}, one NCCL all-reduce of [B,C+1,H,W] sums per forward",
                "l2": "256 MiB buffer written between timed steps"}
    return {"workload": f"{cfg.name}: B={cfg.B} per GPU, N={cfg.N}, {cfg.H}x{cfg.W}, C={cfg.C}, fp32, "
                        f"MSE loss, fwd+bwd", "B_per_gpu": cfg.B, "global_batch": cfg.B * n_gpus, "N": cfg.N,
            "H": cfg.H, "W": cfg.W, "C": cfg.C, "parallelism": f"batch-sharded x{n_gpus}, no collective",
            "l2": "256 MiB buffer written between timed steps"}


# ---------------------------------------------------------------------------
# B200 arm
# ---------------------------------------------------------------------------
def run_b200(args):
    import torch
    import torch.distributed as dist

    from igs_b200 import _lib, workloads
    from igs_b200.gs2d import gaussian_splatting_2d

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: igs_b200 has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    _lib.set_backward_sort(args.backward_sort)
    if args.no_culling:
        _lib.set_culling(False)

    cfg = workloads.CONFIGS[args.workload]
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)
    names = ("positions", "colors", "scales", "rotations", "alphas")
    by_gaussians = cfg.B == 1 and world > 1
    if by_gaussians:
        # one image: every rank owns a contiguous range of its gaussians and the ranks
        # all-reduce the un-normalised sums (strong scaling, total work fixed)
        from igs_b200 import dist as idist

        lo, hi = idist.gaussian_range(cfg.N, world, rank)
        drawn = workloads.draw(cfg, device="cpu")
        drawn.update({k: drawn[k][:, lo:hi].contiguous() for k in names})
        host = {k: v.pin_memory() for k, v in drawn.items()}

        def gaussian_splatting_2d(*a):  # noqa: F811 - the sharded op has the same signature
            return idist.sharded_gaussian_splatting_2d(*a)
    else:
        # every rank draws its own block of the global batch (different seed per rank)
        cfg_r = workloads.SplatConfig(**{**cfg.__dict__, "seed": cfg.seed + 1000 * rank})
        host = {k: v.pin_memory() for k, v in workloads.draw(cfg_r, device="cpu").items()}
    on_dev = {k: v.to(dev) for k, v in host.items()}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    grads_host = {k: torch.empty_like(host[k]).pin_memory() for k in names}
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()

    def step_resident():
        leaves = [on_dev[k].detach().requires_grad_() for k in names]
        out = gaussian_splatting_2d(*leaves, on_dev["x"], on_dev["y"])
        loss = torch.nn.functional.mse_loss(out, on_dev["target"])
        loss.backward()
        return loss, leaves

    # End to end: every step's inputs come from pinned host memory and its gradients and loss
    # go back there.  The copies of step k+1 are issued on a second stream while step k
    # computes (two device buffers, events in both directions), the way a training loop with
    # a prefetching loader runs; the timed region spans the whole loop, first copy included.
    staged = [{k: torch.empty_like(v) for k, v in on_dev.items()} for _ in range(2)]
    copy_stream = torch.cuda.Stream(dev)
    ready = [torch.cuda.Event() for _ in range(2)]
    free = [torch.cuda.Event() for _ in range(2)]

    def prefetch(i):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(free[i])  # the step that last used this buffer has finished
            for k, v in host.items():
                staged[i][k].copy_(v, non_blocking=True)
            ready[i].record(copy_stream)

    def run_e2e(n):
        """n pipelined steps; returns the device time of the whole loop in ms."""
        main = torch.cuda.current_stream(dev)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        begin.record(main)
        for ev in free:
            ev.record(main)  # both buffers are free, and no copy starts before the clock does
        prefetch(0)
        for s_ in range(n):
            i = s_ % 2
            if s_ + 1 < n:
                prefetch((s_ + 1) % 2)
            flush.zero_()
            main.wait_event(ready[i])
            d = staged[i]
            leaves = [d[k].detach().requires_grad_() for k in names]
            out = gaussian_splatting_2d(*leaves, d["x"], d["y"])
            loss = torch.nn.functional.mse_loss(out, d["target"])
            loss.backward()
            for k, t in zip(names, leaves):
                grads_host[k].copy_(t.grad, non_blocking=True)
            loss_host.copy_(loss.detach(), non_blocking=True)
            free[i].record(main)
        end.record(main)
        barrier()
        return begin.elapsed_time(end)

    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = sum(v.numel() * v.element_size() for v in grads_host.values()) + 4

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        """n steps, each bracketed by CUDA events on the current stream, L2 flushed in
        between (outside the events); returns the per-step device times in ms."""
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        barrier()
        for a, b in evs:
            flush.zero_()
            a.record()
            fn()
            b.record()
        barrier()
        return [a.elapsed_time(b) for a, b in evs]

    for _ in range(warmup):
        step_resident()
    probes = _lib.probe_rates(dev) if rank == 0 else None
    barrier()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    _lib.profile_reset()
    _lib.profile_enable(True)
    n0 = _lib.launch_count()
    t_wall0 = time.perf_counter()
    times = timed(step_resident, steps)
    t_wall1 = time.perf_counter()
    launches = _lib.launch_count() - n0
    _lib.profile_enable(False)
    prof = _lib.profile_read()
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None

    for _ in range(2):
        run_e2e(1)
    e2e_total = run_e2e(steps)

    # the kernels' bounded waits report through a status word: one more forward, read it
    probe_fwd = _lib.forward("sr", on_dev["positions"], on_dev["scales"], on_dev["rotations"], None, on_dev["alphas"],
                             on_dev["colors"], on_dev["x"][:, 0], on_dev["y"][:, 0], 1e-6, keep_workspace=True)
    if _lib.read_status(probe_fwd[2]) != 0:
        raise SystemExit("igs_b200: a kernel reported a timed-out wait (status word non-zero)")
    # third word of the status area: gaussians the prologue counted as narrow; the culling
    # instantiations run when that is at least one gaussian in eight
    n_narrow = int(probe_fwd[2][:16].view(torch.int32)[2])
    n_local = host["positions"].shape[0] * host["positions"].shape[1]
    culling = {"enabled": not args.no_culling, "narrow_gaussians": n_narrow, "gaussians": n_local,
               "active": (not args.no_culling) and n_narrow * 8 >= n_local,
               "backward_sort": args.backward_sort,
               "note": "lossless: skipped terms are exact zeros; value counts all B*N*H*W evaluations"}
    if culling["active"]:
        # one backward through the library call, with the order the policy would pass, to read
        # how many (gaussian, pixel) evaluations the culling kernels really did
        x3, y3 = on_dev["x"][:, 0], on_dev["y"][:, 0]
        sorted_bwd = args.backward_sort != "off"
        order = _lib.spatial_order(on_dev["positions"], x3, y3) if sorted_bwd else None
        _lib.set_backward_sort("off")
        probe_bwd = _lib.backward("sr", on_dev["positions"], on_dev["scales"], on_dev["rotations"], None,
                                  on_dev["alphas"], on_dev["colors"], x3, y3, probe_fwd[1], probe_fwd[0],
                                  torch.ones_like(probe_fwd[0]), 1e-6, 0, False, keep_workspace=True, order=order)
        _lib.set_backward_sort(args.backward_sort)
        dense = n_local * cfg.H * cfg.W
        ex_f, ex_b = _lib.read_executed(probe_fwd[2]), _lib.read_executed(probe_bwd["_workspace"])
        culling["executed_evals"] = {"forward": ex_f or dense, "backward": ex_b or dense, "dense": dense}
        culling["executed_share"] = {"forward": (ex_f or dense) / dense, "backward": (ex_b or dense) / dense}
        del probe_bwd
    del probe_fwd

    total_ms = torch.tensor([sum(times), e2e_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    total_ms = total_ms.tolist()
    # evaluations one rank does per step, and the whole job's
    ev_rank = workloads.evals(cfg, N=host["positions"].shape[1])
    ev_job = workloads.evals(cfg) if by_gaussians else ev_rank * world
    value = ev_job * steps / (total_ms[0] * 1e-3)
    e2e_value = ev_job * steps / (total_ms[1] * 1e-3)

    if rank == 0:
        C = cfg.C
        sm = (clocks or {}).get("sm_mhz")
        n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
        # the FMA pipe's measured issue rate: the better of the scalar and the packed probe
        fp32_peak = max(probes["fp32_scalar_lane_instr_per_s"], probes["fp32_packed_lane_instr_per_s"])
        mix_ceiling = {"forward": probes["fp32_forward_mix_lane_instr_per_s"],
                       "backward": probes["fp32_backward_mix_lane_instr_per_s"]}
        # The workloads sample on xy_grid, which the library detects on the device as a
        # separable grid (x by column, y by row) and serves with kernels that share the
        # row / column terms: they ISSUE fewer FMA-pipe instructions per evaluation than the
        # canonical count for arbitrary sample points (fwd 9+C, bwd 18+2C).  `frac` follows
        # the canonical count, so it can exceed 1; `executed_frac` is the pipe's utilisation.
        separable = (os.environ.get("IGS_B200_NO_SEPARABLE") != "1" and C <= 4 and cfg.H >= 4 and cfg.W >= 16)
        # (with more than 4 channels only the forward has a separable instantiation: counted as general)
        if separable:
            executed = {"forward": 5 + C, "backward": 8 + 2 * C}
        else:
            executed = {"forward": 8 + C, "backward": 16 + 2 * C}
        instr = {"forward": 9 + C, "backward": 18 + 2 * C}
        suffix = "_sep" if separable else ""

        share = culling.get("executed_share", {"forward": 1.0, "backward": 1.0})
        if culling["active"]:
            # the headline counts all B*N*H*W evaluations; this is the rate of those really done
            # (forward and backward weighted by their canonical instruction counts)
            w = (share["forward"] * (9 + C) + share["backward"] * (18 + 2 * C)) / (27 + 3 * C)
            culling["executed_evals_per_s"] = value * w
            culling["culled_share"] = 1.0 - w

        def kernel_roof(name):
            ms, n = prof[name]
            if n == 0:
                return None
            # device time of this kernel per pass (with the on-device grid check, the
            # instantiation that does not match returns at once; its launch is included)
            per_pass_s = ms / steps * 1e-3
            # evaluations really done: all of them, or what the culling kernel reports it kept
            ach = ev_rank * share[name] * instr[name] / per_pass_s
            return {"bound": "fp32_fma_pipe", "kernel": f"splat_{name}{suffix}_kernel", "achieved": ach / 1e12,
                    "peak": fp32_peak / 1e12, "unit": "T lane-instr/s", "frac": ach / fp32_peak,
                    "evaluations_counted": "all B*N*H*W" if share[name] == 1.0 else
                    f"executed only: {100 * share[name]:.2f} % of B*N*H*W (the rest are exact zeros, skipped)",
                    "launch_ms": ms / steps, "launches": n,
                    "algorithmic_instr_per_eval": instr[name],
                    "executed_instr_per_eval": executed[name],
                    # with culling active only the evaluations the kernel did not skip are issued
                    # (the culling kernels count them)
                    "executed_frac": ev_rank * share[name] * executed[name] / per_pass_s / fp32_peak,
                    "mix_ceiling_frac": None if separable else mix_ceiling[name] / fp32_peak,
                    "grid": "separable (xy_grid), detected on the device" if separable else "general",
                    "peak_source": "measured live: FFMA-only kernel, best of scalar and f32x2 (igs_probe_fp32_rate)",
                    "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(cfg.name + suffix, {}).get(name)}

        roof = kernel_roof("backward")
        roof_f = kernel_roof("forward")
        step_ach = ev_rank * (share["forward"] * (9 + C) + share["backward"] * (18 + 2 * C)) \
            / (statistics.mean(times) * 1e-3)
        hbm_bytes = (2 * cfg.B * cfg.N * (6 + C) * 4 + 2 * cfg.B * cfg.H * cfg.W * 4 + cfg.B * (C + 1) * cfg.H * cfg.W * 4
                     + cfg.B * (2 * C + 3) * cfg.H * cfg.W * 4 + cfg.B * cfg.N * (6 + C) * 4)
        peaks = {}
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
        except OSError:
            pass
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": total_ms[0] / steps, "higher_is_better": True,
            "scaling": "strong" if by_gaussians else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": workload_config(cfg, world, by_gaussians),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": total_ms[1] / steps,
                    "timing": "whole loop of `steps` steps incl. the first copy; the inputs of step k+1 are copied "
                              "on a second stream while step k computes"},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": roof,
            "roofline_forward": roof_f,
            "roofline_step": {"bound": "fp32_fma_pipe", "achieved": step_ach / 1e12, "peak": fp32_peak / 1e12,
                              "unit": "T lane-instr/s", "frac": step_ach / fp32_peak,
                              "algorithmic_instr_per_eval": 27 + 3 * C,
                              "executed_instr_per_eval": executed["forward"] + executed["backward"],
                              "executed_frac": step_ach / fp32_peak * (share["forward"] * executed["forward"]
                                                                       + share["backward"] * executed["backward"])
                              / (share["forward"] * (9 + C) + share["backward"] * (18 + 2 * C)),
                              "nominal_peak": n_sm * 128 * (sm or 0) * 1e6 / 1e12 if sm else None},
            "probes": probes,
            "hbm": {"algorithmic_bytes_per_step": hbm_bytes,
                    "achieved_gbs": hbm_bytes / (statistics.mean(times) * 1e-3) / 1e9,
                    "peak_gbs": peaks.get("hbm_gbs"), "note": "not the bound: the path is FP32/MUFU issue-bound"},
            "kernel_ms_per_step": {k: v[0] / steps for k, v in prof.items() if v[1]},
            "culling": culling,
            "plan": _lib.describe_plan(cfg.B, host["positions"].shape[1], cfg.H, cfg.W, cfg.C, dev),
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = run_cpu_baseline(cfg, args.cpu_seconds)
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


_RESULT_FD = None


def emit(line):
    """The one JSON line of the run, on the process's original stdout."""
    text = json.dumps(line) + "\n"
    if _RESULT_FD is None:
        sys.stdout.write(text)
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, text.encode())


def main():
    global _RESULT_FD
    args = parse_args()
    # Libraries write to stdout too (NCCL prints its version there when it initialises): keep
    # the original stdout for the result line and send everything else to stderr.
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
