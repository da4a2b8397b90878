"""Benchmark of the splat hot path: gaussian x pixel evaluations per second, forward +
backward, on the batched training shape (B=16, N=8192, 256x256, C=3, fp32).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl reference]

For N > 1 launch under torchrun (one rank per GPU).  The work is FIXED and split over the
ranks (strong scaling): a batch of at least N elements is cut into contiguous blocks
(16 -> 16/N per GPU, no data-path collective); a single image (B = 1) is cut into
gaussian ranges whose un-normalised sums are all-reduced (NCCL) before normalisation.
With the default workload an N > 1 run also times that second scheme on the single-image
configuration and checks its image and gradients against the whole problem rendered on
rank 0 alone (key ``sharded_b1``).

One JSON line is printed by rank 0.  ``value`` is measured with inputs resident on the
device; ``e2e`` is the same metric through the public API from pinned host buffers with
host<->device copies inside the timed region.  ``--impl reference`` times the reference's
CPU path on the host cores instead (its own package where a copy is present under
oracle/_ref, else the torch restatement of it).
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

# dram__bytes_read.sum + dram__bytes_write.sum per launch, from ncu captures of these
# workloads (workload -> kernel -> bytes); None where no capture was taken
NCU_DRAM_BYTES_PER_LAUNCH = {
    "cfg2": {"forward": 18.93e6 + 8.23e6, "backward": 31.38e6 + 8.05e6},
    "cfg2_sep": {"forward": 6.90e6 + 8.56e6, "backward": 26.76e6 + 1.99e6},
    "cfg2_small": {"forward": 3.46e6 + 0.01e6, "backward": 7.03e6},
    "cfg2_small_sep": {"forward": 0.98e6 + 0.02e6, "backward": 5.98e6},
}

METRIC = "gaussian_pixel_evals_per_s_fwd_bwd"
UNIT = "evals/s"
SPLAT_WORKLOADS = ["cfg0", "cfg2", "cfg2_small", "cfg3", "cfg4_small", "cfg4_b8", "cfg4", "narrow", "narrow64k"]
NAMES = ("positions", "colors", "scales", "rotations", "alphas")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg2", choices=SPLAT_WORKLOADS + ["cfg1", "fit"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-culling", action="store_true", help="switch the lossless culling off (for comparison)")
    ap.add_argument("--backward-sort", choices=["auto", "on", "off"], default="auto",
                    help="spatial processing order of the gaussians (results are the same bits)")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="budget of the CPU baseline leg")
    ap.add_argument("--warped-grid", action="store_true",
                    help="move one sample point off the pixel grid: the grid is then not separable and the "
                         "general kernels (arbitrary sample points) run instead of the separable ones")
    ap.add_argument("--no-sharded-leg", action="store_true",
                    help="N > 1, default workload: skip the extra single-image gaussian-sharded leg")
    ap.add_argument("--sharded-steps", type=int, default=20)
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
# CPU arm: the reference's chunked torch path on the host cores
# ---------------------------------------------------------------------------
def cpu_config(workload):
    """The splat configuration whose CPU cost stands beside a workload (the module and the
    fit loop render the same op: their splat shape is what the CPU arm times)."""
    from igs_b200 import workloads

    if workload == "cfg1":
        return workloads.SplatConfig("cfg1", 1, 4096, 256, 256, 3, 0.02, 0.2, seed=1)
    if workload == "fit":
        return workloads.SplatConfig("fit", 1, FIT_N, FIT_SIZE, FIT_SIZE, 3, 0.004, 0.012, seed=9)
    return workloads.CONFIGS[workload]


def cpu_step_fn(cfg, n_sample, threads):
    """Returns (step callable, evals per step, description, kind).  The sample keeps the full
    batch and the full image and takes the first n_sample gaussians (a multiple of the
    reference's chunk of 32): the reference's loop runs N/32 identical iterations over
    [B,32,H,W] blocks, so the sample has the working set and the evals/s of the whole
    workload.  kind "reference": the reference's own package (a copy under oracle/_ref); "port":
    its torch restatement, used where no copy is present."""
    import torch

    from igs_b200 import workloads
    from oracle import ref_copy

    torch.set_num_threads(threads)
    d = workloads.draw(cfg, N=n_sample, device="cpu")

    def gout(o):
        return 2 * (o - d["target"]) / o.numel()

    if ref_copy.available():
        mod = ref_copy.load()

        def step():
            return ref_copy.render_fwd_bwd(mod, d["positions"], d["colors"], d["scales"], d["rotations"], d["alphas"],
                                           d["x"], d["y"], gout)[1]
        kind, what = "reference", ("the reference's own chunked torch Function (src/igs/gs2d.py:265-465 behind "
                             "gaussian_splatting_2d), from the copy under oracle/_ref")
    else:
        from oracle import chunked_port as cp

        def step():
            return cp.render_fwd_bwd(d["positions"], d["colors"], d["scales"], d["rotations"], d["alphas"], d["x"],
                                     d["y"], gout)[1]
        kind, what = "port", ("torch restatement of the reference's chunked path (oracle/chunked_port.py; no copy "
                              "of the reference under oracle/_ref here)")
    sample = f"full batch B={cfg.B}, first {n_sample} of {cfg.N} gaussians, full {cfg.H}x{cfg.W} image; {what}"
    return step, cfg.B * n_sample * cfg.H * cfg.W, sample, kind


def calibrate_cpu_sample(cfg, threads, target_s):
    """Gaussians per CPU step so that one step takes about target_s seconds."""
    step, ev, _, _ = cpu_step_fn(cfg, 32, threads)
    step()
    t0 = time.perf_counter()
    step()
    dt = max(time.perf_counter() - t0, 1e-4)
    n = int(32 * target_s / dt) // 32 * 32
    return max(32, min(cfg.N, n))


def run_cpu_baseline(cfg, seconds):
    threads = os.cpu_count() or 1
    n = calibrate_cpu_sample(cfg, threads, max(seconds / 4.0, 0.5))
    step, ev, sample, kind = cpu_step_fn(cfg, n, threads)
    step()  # warm-up
    times = []
    t_end = time.perf_counter() + seconds * 0.6
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 10):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    res = {"value": ev / med, "unit": UNIT, "cores": threads, "kind": kind, "cpu_sample_N": n,
           "sample": f"{sample}; median of {len(times)} steps of {med:.2f} s"}
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
    """`--impl reference`: the reference's CPU path on the host cores, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = cpu_config(args.workload)
    threads = os.cpu_count() or 1
    # size each step to ~1.5 s so that steps + warm-ups stay within a few minutes
    budget = 150.0 / max(args.steps + args.warmup, 1)
    n = calibrate_cpu_sample(cfg, threads, min(1.5, budget))
    step, ev, sample, kind = cpu_step_fn(cfg, n, threads)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = ev * args.steps / dt
    config = splat_config_dict(cfg, args.gpus, "gaussians" if cfg.B < args.gpus else "batch")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config, "cpu_sample_N": n,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "cpu_sample_N": n,
                         "sample": f"each step: {sample}; quoted as a rate (the cost is linear in the chunks of 32 "
                                   "gaussians)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def splat_config_dict(cfg, n_gpus, split):
    """`config` of the JSON line.  split: "batch" (contiguous blocks of the batch per GPU) or
    "gaussians" (contiguous ranges of the gaussians per GPU + one all-reduce)."""
    base = {"N": cfg.N, "H": cfg.H, "W": cfg.W, "C": cfg.C, "global_batch": cfg.B,
            "l2": "256 MiB buffer written between timed steps"}
    if split == "gaussians" and n_gpus > 1:
        base.update({
            "workload": f"{cfg.name}: B={cfg.B}, N={cfg.N} split over {n_gpus} GPUs, {cfg.H}x{cfg.W}, C={cfg.C}, fp32, "
                        f"MSE loss, fwd+bwd",
            "B_per_gpu": cfg.B, "N_per_gpu": cfg.N / n_gpus,
            "parallelism": f"gaussian ranges x{n_gpus}, one NCCL all-reduce of [B,C+1,H,W] sums per forward"})
    else:
        base.update({
            "workload": f"{cfg.name}: B={cfg.B}" + (f" split over {n_gpus} GPUs" if n_gpus > 1 else "")
                        + f", N={cfg.N}, {cfg.H}x{cfg.W}, C={cfg.C}, fp32, MSE loss, fwd+bwd",
            "B_per_gpu": cfg.B / n_gpus, "N_per_gpu": cfg.N,
            "parallelism": f"batch blocks x{n_gpus}, no collective" if n_gpus > 1 else "one GPU"})
    return base


# ---------------------------------------------------------------------------
# workloads of the B200 arm: host tensors + a step over device tensors
# ---------------------------------------------------------------------------
FIT_N, FIT_SIZE = 16384, 1024


class SplatWorkload:
    """gaussian_splatting_2d forward + MSE + backward on one of the seeded configurations;
    with several ranks, this rank's share of the FIXED global problem."""

    def __init__(self, cfg, rank, world, dev, torch):
        from igs_b200 import dist as idist
        from igs_b200 import workloads

        self.cfg, self.C = cfg, cfg.C
        self.split = "gaussians" if (cfg.B < world) else "batch"
        drawn = workloads.draw(cfg, device="cpu")
        if world > 1 and self.split == "gaussians":
            lo, hi = idist.gaussian_range(cfg.N, world, rank)
            drawn.update({k: drawn[k][:, lo:hi].contiguous() for k in NAMES})
        elif world > 1:
            lo, hi = idist.batch_range(cfg.B, world, rank)
            drawn = {k: v[lo:hi].contiguous() for k, v in drawn.items()}
        self.range = (lo, hi) if world > 1 else None
        self.host = {k: v.pin_memory() for k, v in drawn.items()}
        self.B_local, self.N_local = drawn["positions"].shape[:2]
        self.evals_rank = self.B_local * self.N_local * cfg.H * cfg.W
        self.evals_job = cfg.B * cfg.N * cfg.H * cfg.W
        self.sharded = world > 1 and self.split == "gaussians"
        self.separable_grid = cfg.H >= 4 and cfg.W >= 16
        self.grad_names = NAMES
        self.torch = torch

    def config(self, world):
        return splat_config_dict(self.cfg, world, self.split)

    def step(self, t):
        """One forward + backward on the device tensors t; returns (loss, gradients)."""
        torch = self.torch
        leaves = [t[k].detach().requires_grad_() for k in NAMES]
        if self.sharded:
            from igs_b200.dist import sharded_gaussian_splatting_2d as render
        else:
            from igs_b200.gs2d import gaussian_splatting_2d as render
        out = render(*leaves, t["x"], t["y"])
        loss = torch.nn.functional.mse_loss(out, t["target"])
        loss.backward()
        return loss, [v.grad for v in leaves]


class ModuleWorkload:
    """BASELINE configuration 1: GaussianSplatting2D(32 gaussians per feature, feature_dim
    1024) on x ~ N(0,1) [1,128,1024] -> 4096 gaussians at 256x256, forward + MSE + backward
    through the module (Linear layer included)."""

    def __init__(self, rank, world, dev, torch):
        from igs_b200 import GaussianSplatting2D

        if world > 1:
            raise SystemExit("the module workload runs on one GPU")
        torch.manual_seed(1)
        self.module = GaussianSplatting2D(32, 1024).to(dev)
        gen = torch.Generator().manual_seed(1)
        self.host = {"feature": torch.randn(1, 128, 1024, generator=gen).pin_memory(),
                     "target": torch.rand(1, 3, 256, 256, generator=gen).pin_memory()}
        self.cfg = cpu_config("cfg1")
        self.C, self.B_local, self.N_local = 3, 1, 4096
        self.evals_rank = self.evals_job = 4096 * 256 * 256
        self.split, self.sharded, self.separable_grid, self.range = "batch", False, True, None
        self.grad_names = ("feature", "proj.weight", "proj.bias")
        self.torch = torch

    def config(self, world):
        return {"workload": "cfg1: GaussianSplatting2D(32, 1024) module on x[1,128,1024] -> N=4096 gaussians, "
                            "256x256, C=3, fp32, MSE loss, fwd+bwd through the module",
                "N": 4096, "H": 256, "W": 256, "C": 3, "global_batch": 1, "B_per_gpu": 1, "N_per_gpu": 4096,
                "parallelism": "one GPU", "l2": "256 MiB buffer written between timed steps"}

    def step(self, t):
        torch = self.torch
        self.module.zero_grad(set_to_none=True)
        x = t["feature"].detach().requires_grad_()
        out, _ = self.module(x, size=(256, 256))
        loss = torch.nn.functional.mse_loss(out, t["target"])
        loss.backward()
        return loss, [x.grad, self.module.proj.weight.grad, self.module.proj.bias.grad]


class FitWorkload:
    """One eager Adam step of the per-image fit (igs_b200.fit.ImageFitter): FIT_N free
    gaussians of scale e^-5 in shuffled order against a FIT_SIZE^2 target; render + MSE +
    backward + optimiser step."""

    def __init__(self, rank, world, dev, torch):
        from igs_b200 import fit

        if world > 1:
            raise SystemExit("the fit workload runs on one GPU")
        gen = torch.Generator().manual_seed(9)
        self.fit = fit
        self.model = fit.ImageFitter(FIT_N, 3, init_log_scale=-5.0)
        perm = torch.randperm(FIT_N, generator=gen)
        with torch.no_grad():
            self.model.position.copy_(self.model.position[:, perm])
        self.model.to(dev)
        self.opt = torch.optim.Adam(self.model.parameters(), lr=1e-2, fused=True)
        self.host = {"target": torch.rand(1, 3, FIT_SIZE, FIT_SIZE, generator=gen).pin_memory()}
        self.cfg = cpu_config("fit")
        self.C, self.B_local, self.N_local = 3, 1, FIT_N
        self.evals_rank = self.evals_job = FIT_N * FIT_SIZE * FIT_SIZE
        self.split, self.sharded, self.separable_grid, self.range = "batch", False, True, None
        self.grad_names = ("position", "log_scale", "rotation", "color")
        self.torch = torch

    def config(self, world):
        return {"workload": f"fit: ImageFitter with {FIT_N} free gaussians (log-scale -5, shuffled), "
                            f"{FIT_SIZE}x{FIT_SIZE}, C=3, fp32; render + MSE + backward + Adam step, eager",
                "N": FIT_N, "H": FIT_SIZE, "W": FIT_SIZE, "C": 3, "global_batch": 1, "B_per_gpu": 1,
                "N_per_gpu": FIT_N, "parallelism": "one GPU", "l2": "256 MiB buffer written between timed steps"}

    def step(self, t):
        loss = self.fit._eager_step(self.model, self.opt, t["target"])
        m = self.model
        return loss, [m.position.grad, m.log_scale.grad, m.rotation.grad, m.color.grad]


def make_workload(name, rank, world, dev, torch):
    from igs_b200 import workloads

    if name == "cfg1":
        return ModuleWorkload(rank, world, dev, torch)
    if name == "fit":
        return FitWorkload(rank, world, dev, torch)
    return SplatWorkload(workloads.CONFIGS[name], rank, world, dev, torch)


# ---------------------------------------------------------------------------
# B200 arm
# ---------------------------------------------------------------------------
def run_b200(args):
    import torch
    import torch.distributed as dist

    from igs_b200 import _lib

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

    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)
    wl = make_workload(args.workload, rank, world, dev, torch)
    if args.warped_grid:
        if "x" not in wl.host:
            raise SystemExit("--warped-grid applies to the workloads that pass their own sample grid")
        wl.host["x"][0, 0, 0, 0] += 1e-3
        wl.separable_grid = False
    host = wl.host
    on_dev = {k: v.to(dev) for k, v in host.items()}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

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

    def step_resident():
        return wl.step(on_dev)

    # End to end: every step's inputs come from pinned host memory and its gradients and loss
    # go back there.  The copies of step k+1 are issued on a second stream while step k
    # computes (two device buffers, events in both directions), the way a training loop with
    # a prefetching loader runs; the timed region spans the whole loop, first copy included.
    staged = [{k: torch.empty_like(v) for k, v in on_dev.items()} for _ in range(2)]
    copy_stream = torch.cuda.Stream(dev)
    ready = [torch.cuda.Event() for _ in range(2)]
    free = [torch.cuda.Event() for _ in range(2)]
    _, g0 = step_resident()
    grads_host = [torch.empty(g.shape, dtype=g.dtype).pin_memory() for g in g0]
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()
    del g0

    def prefetch(i):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(free[i])  # the step that last used this buffer has finished
            for k, v in host.items():
                staged[i][k].copy_(v, non_blocking=True)
            ready[i].record(copy_stream)

    d2h_stream = torch.cuda.Stream(dev)

    def run_e2e(n):
        """n pipelined steps; returns the device time of the whole loop in ms.  The gradients
        and the loss of step k go back to pinned host memory on a third stream while step k+1
        computes; the clock stops when the last of them has arrived."""
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
            loss, grads = wl.step(staged[i])
            computed = torch.cuda.Event()
            computed.record(main)
            free[i].record(main)
            with torch.cuda.stream(d2h_stream):
                d2h_stream.wait_event(computed)
                for h, g in zip(grads_host, grads):
                    h.copy_(g, non_blocking=True)
                    g.record_stream(d2h_stream)
                loss_d = loss.detach()
                loss_host.copy_(loss_d, non_blocking=True)
                loss_d.record_stream(d2h_stream)
        main.wait_stream(d2h_stream)
        end.record(main)
        barrier()
        return begin.elapsed_time(end)

    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = sum(v.numel() * v.element_size() for v in grads_host) + 4

    sampler = ClockSampler(local_rank) if rank == 0 else None  # (nvidia-smi needs a moment to start)
    for _ in range(warmup):
        step_resident()
    probes = None
    if rank == 0:
        from igs_b200 import probes as probe_lib

        probes = probe_lib.rates(dev.index)
    barrier()

    # Timed region: `steps` steps; the two splat kernels are bracketed by event pairs on their
    # own stream inside it (the roofline's launch durations), the small kernels are not: an
    # event pair costs a few microseconds per launch, which a sub-millisecond step notices.
    _lib.profile_reset()
    _lib.profile_enable(2)
    n0 = _lib.launch_count()
    t_wall0 = time.perf_counter()
    times = timed(step_resident, steps)
    launches = _lib.launch_count() - n0
    _lib.profile_enable(False)
    prof = _lib.profile_read()
    # the same steps with every kernel bracketed (the per-kernel breakdown) ...
    _lib.profile_reset()
    _lib.profile_enable(1)
    timed(step_resident, steps)
    _lib.profile_enable(False)
    prof_all = _lib.profile_read()
    # ... and with no event pairs at all
    times_plain = timed(step_resident, steps)
    # clocks: the samples taken while these three passes of the same steps ran (a strong-scaled
    # timed pass alone can be shorter than nvidia-smi's sampling period)
    clocks = sampler.stop(t_wall0, time.perf_counter()) if sampler else None
    if clocks is not None:
        clocks["window"] = "the timed pass and two more passes of the same steps right behind it"

    for _ in range(2):
        run_e2e(1)
    e2e_total = run_e2e(steps)
    # how long one step's host->device copies take by themselves while every rank copies at
    # once (they overlap the previous step's kernels unless they take longer than a step)
    barrier()
    ca, cb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for ev in free:
        ev.record(torch.cuda.current_stream(dev))
    with torch.cuda.stream(copy_stream):
        ca.record(copy_stream)
    for i in range(4):
        prefetch(i % 2)
    with torch.cuda.stream(copy_stream):
        cb.record(copy_stream)
    barrier()
    h2d_copy_ms = ca.elapsed_time(cb) / 4

    culling = None
    if isinstance(wl, SplatWorkload):
        culling = culling_report(args, wl, on_dev, _lib, torch)

    total_ms = torch.tensor([sum(times), e2e_total, sum(times_plain), h2d_copy_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    total_ms = total_ms.tolist()
    value = wl.evals_job * steps / (total_ms[0] * 1e-3)
    e2e_value = wl.evals_job * steps / (total_ms[1] * 1e-3)

    sharded_b1 = None
    if world > 1 and args.workload == "cfg2" and not args.no_sharded_leg:
        sharded_b1 = sharded_single_image_leg(args, rank, world, dev, torch, dist, timed, barrier)

    if rank == 0:
        C = wl.C
        sm = (clocks or {}).get("sm_mhz")
        n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
        ev_rank = wl.evals_rank
        # the FMA pipe's measured issue rate: the better of the scalar and the packed probe
        fp32_peak = max(probes["fp32_scalar_lane_instr_per_s"], probes["fp32_packed_lane_instr_per_s"])
        mix_ceiling = {"forward": probes["fp32_forward_mix_lane_instr_per_s"],
                       "backward": probes["fp32_backward_mix_lane_instr_per_s"]}
        # The workloads sample on xy_grid, which the library detects as a separable grid (x by
        # column, y by row) and serves with kernels that share the row / column terms: they
        # ISSUE fewer FMA-pipe instructions per evaluation than the canonical count for
        # arbitrary sample points (fwd 9+C, bwd 18+2C).  `frac` follows the canonical count,
        # so it can exceed 1; `executed_frac` is the pipe's utilisation.
        has_sep_f, has_sep_b = _lib.separable_kernels(C)
        sep_f, sep_b = wl.separable_grid and has_sep_f, wl.separable_grid and has_sep_b
        # (separable: forward 4.5 + C; backward 7 + 2C in the pixel-packed kernels for up to 4
        # channels, which share dx and dx^2 between the two rows of a block, 8 + 2C in the
        # row-streaming 8 / 16-channel ones)
        executed = {"forward": (4.5 + C) if sep_f else (8 + C),
                    "backward": ((7 if C <= 4 else 8) + 2 * C) if sep_b else (16 + 2 * C)}
        instr = {"forward": 9 + C, "backward": 18 + 2 * C}
        sep = {"forward": sep_f, "backward": sep_b}

        share = (culling or {}).get("executed_share", {"forward": 1.0, "backward": 1.0})
        if culling and culling["active"]:
            # the headline counts all B*N*H*W evaluations; this is the rate of those really done
            # (forward and backward weighted by their canonical instruction counts)
            w = (share["forward"] * (9 + C) + share["backward"] * (18 + 2 * C)) / (27 + 3 * C)
            culling["executed_evals_per_s"] = value * w
            culling["culled_share"] = 1.0 - w

        def kernel_roof(name):
            ms, n = prof[name]
            if n == 0:
                return None
            # device time of this kernel per pass (instantiations that the data does not call
            # for return at once; their launches are included)
            per_pass_s = ms / steps * 1e-3
            # evaluations really done: all of them, or what the culling kernel reports it kept
            ach = ev_rank * share[name] * instr[name] / per_pass_s
            suffix = "_sep" if sep[name] else ""
            return {"bound": "fp32_fma_pipe", "kernel": f"splat_{name}{suffix}_kernel", "achieved": ach / 1e12,
                    "peak": fp32_peak / 1e12, "unit": "T lane-instr/s", "frac": ach / fp32_peak,
                    "evaluations_counted": ("all B*N*H*W; this workload's gaussians are narrow and the kernels skip "
                                            "most evaluations, whose executed share is not read here: the fractions "
                                            "are no utilisation figures") if culling is None else
                    "all B*N*H*W" if share[name] == 1.0 else
                    f"executed only: {100 * share[name]:.2f} % of B*N*H*W (the rest are exact zeros, skipped)",
                    "launch_ms": ms / steps, "launches": n,
                    "algorithmic_instr_per_eval": instr[name],
                    "executed_instr_per_eval": executed[name],
                    "executed_frac": ev_rank * share[name] * executed[name] / per_pass_s / fp32_peak,
                    "mix_ceiling_frac": None if sep[name] else mix_ceiling[name] / fp32_peak,
                    # f32x2 FMAs with three distinct register operands (every accumulation is one)
                    # issue at this fraction of the FFMA-only rate: the register file's limit
                    "three_operand_ceiling_frac": probes["fp32_packed_3operand_lane_instr_per_s"] / fp32_peak,
                    "grid": "separable (xy_grid)" if sep[name] else "general",
                    "peak_source": "measured live: FFMA-only kernel, best of scalar and f32x2 (igs_b200.probes)",
                    "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(args.workload + suffix, {}).get(name)
                    if world == 1 else None}

        roof = kernel_roof("backward")
        roof_f = kernel_roof("forward")
        mean_s = statistics.mean(times) * 1e-3
        step_ach = ev_rank * (share["forward"] * (9 + C) + share["backward"] * (18 + 2 * C)) / mean_s
        cfg = wl.cfg
        B, N = wl.B_local, wl.N_local
        hbm_bytes = (2 * B * N * (6 + C) * 4 + 2 * B * cfg.H * cfg.W * 4 + B * (C + 1) * cfg.H * cfg.W * 4
                     + B * (2 * C + 3) * cfg.H * cfg.W * 4 + B * N * (6 + C) * 4)
        peaks = {}
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
        except OSError:
            pass
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": total_ms[0] / steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": wl.config(world),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": total_ms[1] / steps,
                    "h2d_copy_ms_per_step": total_ms[3],
                    "h2d_gbs_per_gpu": h2d / (total_ms[3] * 1e-3) / 1e9 if total_ms[3] > 0 else None,
                    "timing": "whole loop of `steps` steps incl. the first copy in and the last copy out; the inputs "
                              "of step k+1 are copied on a second stream and the results of step k-1 on a third "
                              "while step k computes"},
            "gpu_launches": launches,
            "launches_per_step": launches / steps,
            "ms_per_step_without_kernel_events": total_ms[2] / steps,
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
            "hbm": {"algorithmic_bytes_per_step": hbm_bytes, "achieved_gbs": hbm_bytes / mean_s / 1e9,
                    "peak_gbs": peaks.get("hbm_gbs"), "note": "not the bound: the path is FP32/MUFU issue-bound"},
            "kernel_ms_per_step": {k: v[0] / steps for k, v in prof_all.items() if v[1]},
            "culling": culling,
            "plan": _lib.describe_plan(B, N, cfg.H, cfg.W, C, dev),
        }
        if sharded_b1 is not None:
            line["sharded_b1"] = sharded_b1
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = run_cpu_baseline(cpu_config(args.workload), args.cpu_seconds)
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def culling_report(args, wl, on_dev, _lib, torch):
    """Reads the status words of one more forward (bounded waits, narrow-gaussian count) and,
    when the culling kernels are the ones that run, how many evaluations they really did."""
    x3, y3 = on_dev["x"][:, 0], on_dev["y"][:, 0]
    probe_fwd = _lib.forward("sr", on_dev["positions"], on_dev["scales"], on_dev["rotations"], None, on_dev["alphas"],
                             on_dev["colors"], x3, y3, 1e-6, keep_workspace=True)
    if _lib.read_status(probe_fwd[2]) != 0:
        raise SystemExit("igs_b200: a kernel reported a timed-out wait (status word non-zero)")
    # third word of the status area: gaussians the prologue counted as narrow; the culling
    # instantiations run when that is at least one gaussian in eight
    n_narrow = int(probe_fwd[2][:16].view(torch.int32)[2])
    n_local = wl.B_local * wl.N_local
    culling = {"enabled": not args.no_culling, "narrow_gaussians": n_narrow, "gaussians": n_local,
               "active": (not args.no_culling) and n_narrow * 8 >= n_local,
               "backward_sort": args.backward_sort,
               "note": "lossless: skipped terms are exact zeros; value counts all B*N*H*W evaluations"}
    if culling["active"]:
        # one backward through the library call, with the order the policy would pass, to read
        # how many (gaussian, pixel) evaluations the culling kernels really did
        order = None
        if args.backward_sort != "off":  # the order the call layer would pass
            order = _lib.order_by_policy(_lib._shape_memo(x3.device, wl.B_local, wl.N_local, wl.cfg.H, wl.cfg.W),
                                         on_dev["positions"], None, None, x3, y3, on_dev["scales"], False,
                                         on_dev["rotations"])
            if order is None:
                order = _lib.spatial_order(on_dev["positions"], x3, y3)
        probe_bwd = _lib.backward("sr", on_dev["positions"], on_dev["scales"], on_dev["rotations"], None,
                                  on_dev["alphas"], on_dev["colors"], x3, y3, probe_fwd[1], probe_fwd[0],
                                  torch.ones_like(probe_fwd[0]), 1e-6, 0, False, keep_workspace=True, order=order)
        if order is not None:  # the ordered forward is what the steps ran
            probe_fwd = _lib.forward("sr", on_dev["positions"], on_dev["scales"], on_dev["rotations"], None,
                                     on_dev["alphas"], on_dev["colors"], x3, y3, 1e-6, keep_workspace=True,
                                     order=order)
        dense = n_local * wl.cfg.H * wl.cfg.W
        ex_f, ex_b = _lib.read_executed(probe_fwd[2]), _lib.read_executed(probe_bwd["_workspace"])
        culling["executed_evals"] = {"forward": ex_f or dense, "backward": ex_b or dense, "dense": dense}
        culling["executed_share"] = {"forward": (ex_f or dense) / dense, "backward": (ex_b or dense) / dense}
    return culling


def sharded_single_image_leg(args, rank, world, dev, torch, dist, timed, barrier):
    """Second leg of an N > 1 run: the single-image configuration (B=1, N=16384, 512x512)
    split into gaussian ranges, one all-reduce of [B,C+1,H,W] per forward.  Times it (max
    over ranks), then rank 0 renders the WHOLE problem alone: the time gives the speed-up,
    the image and rank 0's slice of the gradients give the parity figure."""
    from igs_b200 import dist as idist
    from igs_b200 import workloads
    from igs_b200.gs2d import gaussian_splatting_2d

    cfg = workloads.CONFIGS["cfg3"]
    n_steps = max(args.sharded_steps, 1)
    full = workloads.draw(cfg, device="cpu")
    lo, hi = idist.gaussian_range(cfg.N, world, rank)
    mine = {k: (full[k][:, lo:hi].contiguous() if k in NAMES else full[k]).to(dev) for k in full}
    result = {}

    def step_sharded():
        leaves = [mine[k].detach().requires_grad_() for k in NAMES]
        out = idist.sharded_gaussian_splatting_2d(*leaves, mine["x"], mine["y"])
        torch.nn.functional.mse_loss(out, mine["target"]).backward()
        result["out"], result["grads"] = out.detach(), [v.grad for v in leaves]

    for _ in range(3):
        step_sharded()
    n0 = _launch_count()
    t_sh = torch.tensor([sum(timed(step_sharded, n_steps))], dtype=torch.float64, device=dev)
    launches = (_launch_count() - n0) / n_steps
    dist.all_reduce(t_sh, op=dist.ReduceOp.MAX)
    ms_sharded = t_sh.item() / n_steps

    report = None
    if rank == 0:
        whole = {k: v.to(dev) for k, v in full.items()}
        one = {}

        def step_one():
            leaves = [whole[k].detach().requires_grad_() for k in NAMES]
            out = gaussian_splatting_2d(*leaves, whole["x"], whole["y"])
            torch.nn.functional.mse_loss(out, whole["target"]).backward()
            one["out"], one["grads"] = out.detach(), [v.grad for v in leaves]

        for _ in range(3):
            step_one()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_steps)]
        torch.cuda.synchronize()
        for a, b in evs:
            a.record()
            step_one()
            b.record()
        torch.cuda.synchronize()
        ms_one = sum(a.elapsed_time(b) for a, b in evs) / n_steps

        def err(a, b):
            return float((a - b).abs().max() / b.abs().max())

        parity = {"image": err(result["out"], one["out"])}
        for k, g_sh, g_one in zip(NAMES, result["grads"], one["grads"]):
            parity["d_" + k] = err(g_sh, g_one[:, lo:hi])
        evals = cfg.B * cfg.N * cfg.H * cfg.W
        report = {"workload": f"cfg3: B=1, N={cfg.N} as {world} gaussian ranges, {cfg.H}x{cfg.W}, C=3, MSE, fwd+bwd; one "
                              "NCCL all-reduce of [1,4,512,512] fp32 (4 MiB) per forward",
                  "steps": n_steps, "ms_per_step": ms_sharded, "value": evals / (ms_sharded * 1e-3), "unit": UNIT,
                  "one_gpu_ms_per_step": ms_one, "speedup_vs_one_gpu": ms_one / ms_sharded,
                  "library_launches_per_step": launches,
                  "parity": parity, "parity_max_err": max(parity.values()),
                  "parity_note": "max|a-b| / max|b| of the all-reduced image and of rank 0's slice of every "
                                 "gradient against the whole problem rendered on rank 0 alone; tolerance 1e-4"}
    barrier()
    return report


def _launch_count():
    from igs_b200 import _lib

    return _lib.launch_count()


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
    # the reference's `render` is wrapped in torch.compile, which its CPU path cannot use;
    # nothing on the B200 arm compiles anything (read when torch._dynamo is first imported)
    os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
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
