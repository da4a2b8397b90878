"""Multi-process tests of igs_b200.dist.

CPU (gloo, world size 2): the host logic of the gaussian-sharded op -- range split,
shape handshake, all-reduce, local backward -- with the device calls replaced by the CPU
oracle (the test supplies that stand-in; the package has no CPU path of its own).
GPU (nccl, needs 2 devices): the same op on the CUDA kernels against the one-GPU result.
"""
import datetime
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests._util import assert_close


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(B, N, H, W, C, seed):
    from igs_b200 import workloads

    cfg = workloads.SplatConfig("t", B, N, H, W, C, 0.1, 0.5, seed=seed)
    return workloads.draw(cfg, device="cpu")


class OracleBackend:
    """CPU stand-in for the three device calls, built on the oracle (tests only)."""

    @staticmethod
    def forward_sums(pos, col, sc, rot, al, x3, y3, eps):
        from oracle import splat_oracle as so

        c00, c01, c11 = so.cov_inv(sc.numpy(), rot.numpy(), eps, np.float64)
        ones = np.ones((*col.shape[:2], 1))
        # un-normalised sums: render with eps=0 and multiply back by the weight sum
        out, wsum = so.forward(x3.numpy(), y3.numpy(), pos.numpy(), c00, c01, c11, al.numpy(),
                               np.concatenate([col.numpy().astype(np.float64), ones], 2), 0.0, np.float64)
        sums = out * wsum[:, None]
        sums[:, -1] = wsum
        return torch.from_numpy(np.nan_to_num(sums).astype(np.float32))

    @staticmethod
    def normalize(sums, eps):
        wsum = sums[:, -1]
        return (sums[:, :-1] / (wsum + eps)[:, None]).contiguous(), wsum.contiguous()

    @staticmethod
    def backward(pos, col, sc, rot, al, x3, y3, wsum, out, gout, eps, grad_mode):
        from oracle import splat_oracle as so

        c00, c01, c11 = so.cov_inv(sc.numpy(), rot.numpy(), eps, np.float64)
        g = so.backward(x3.numpy(), y3.numpy(), pos.numpy(), c00, c01, c11, al.numpy(), col.numpy(), wsum.numpy(),
                        out.numpy(), gout.numpy(), eps, grad_mode, False, np.float64)
        gs, gr = so.cov_inv_backward(sc.numpy(), rot.numpy(), g["c00"], g["c01"], g["c11"], eps, np.float64)
        t = lambda a: torch.from_numpy(np.asarray(a, np.float32))
        return {"positions": t(g["positions"]), "colors": t(g["colors"]), "scales": t(gs), "rotations": t(gr),
                "alphas": t(g["alphas"])}


def _init(rank, world, port, backend, timeout_s=60):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    kw = {}
    if backend == "nccl":
        torch.cuda.set_device(rank)
        kw["device_id"] = torch.device("cuda", rank)
    dist.init_process_group(backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s), **kw)


def _worker_sharded(rank, world, port, backend, q):
    from igs_b200 import dist as idist

    try:
        _init(rank, world, port, backend)
        dev = torch.device("cuda", rank) if backend == "nccl" else torch.device("cpu")
        d = _inputs(1, 203, 20, 24, 3, seed=5)  # 203 gaussians: uneven ranges
        lo, hi = idist.gaussian_range(203, world, rank)
        names = ("positions", "colors", "scales", "rotations", "alphas")
        leaves = [d[k][:, lo:hi].contiguous().to(dev).requires_grad_() for k in names]
        be = None if backend == "nccl" else OracleBackend
        out = idist.sharded_gaussian_splatting_2d(*leaves, d["x"].to(dev), d["y"].to(dev), backend=be)
        loss = ((out - d["target"].to(dev)) ** 2).sum()
        loss.backward()
        q.put((rank, lo, hi, out.detach().cpu().numpy(), [t.grad.cpu().numpy() for t in leaves], None))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # noqa: BLE001 - reported to the parent
        q.put((rank, 0, 0, None, None, repr(exc)))


def _run_sharded(world, backend):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_sharded, args=(r, world, port, backend, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for r in res:
        assert r[5] is None, f"rank {r[0]} failed: {r[5]}"
    return sorted(res, key=lambda r: r[0])


def _single_process_oracle():
    from oracle import splat_oracle as so

    d = {k: v.numpy() for k, v in _inputs(1, 203, 20, 24, 3, seed=5).items()}
    out, _, grads = so.render_with_grads(d["positions"], d["colors"], d["scales"], d["rotations"], d["alphas"],
                                         d["x"][:, 0], d["y"][:, 0], lambda o: 2 * (o - d["target"]), 1e-6,
                                         dtype=np.float64)
    return out, grads


def _check_against_single(res):
    out, grads = _single_process_oracle()
    names = ("positions", "colors", "scales", "rotations", "alphas")
    for rank, lo, hi, o, g, _ in res:
        assert_close(o, out, 1e-4, f"rank {rank} image")
    for i, k in enumerate(names):
        got = np.concatenate([r[4][i] for r in res], axis=1)
        assert_close(got, grads[k], 1e-4, f"d_{k} gathered over ranks")
    assert [(r[1], r[2]) for r in res] == [(0, 102), (102, 203)]


def test_ranges_partition():
    from igs_b200.dist import batch_range, gaussian_range

    for n, w in ((16, 8), (1, 4), (203, 2), (7, 3), (0, 2)):
        parts = [batch_range(n, w, r) for r in range(w)]
        assert parts[0][0] == 0 and parts[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
        assert max(h - l for l, h in parts) - min(h - l for l, h in parts) <= 1
    assert gaussian_range(16384, 8, 3) == (6144, 8192)
    with pytest.raises(ValueError):
        batch_range(4, 2, 2)


def test_gaussian_sharded_two_ranks_gloo():
    _check_against_single(_run_sharded(2, "gloo"))


def _worker_mismatch(rank, world, port, q):
    from igs_b200 import dist as idist

    try:
        _init(rank, world, port, "gloo")
        H = 20 if rank == 0 else 22  # rank 1 was handed another image size
        d = _inputs(1, 40, H, 24, 3, seed=6)
        args = [d[k] for k in ("positions", "colors", "scales", "rotations", "alphas")]
        idist.sharded_gaussian_splatting_2d(*args, d["x"], d["y"], backend=OracleBackend)
        q.put((rank, "no error"))
    except ValueError as exc:
        q.put((rank, "ValueError: " + str(exc)))
    except Exception as exc:  # noqa: BLE001
        q.put((rank, repr(exc)))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_shape_mismatch_raises_on_every_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_mismatch, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert all(v.startswith("ValueError: ranks disagree") for v in res.values()), res


def _worker_peer_dies(rank, world, port, q):
    """Failure made on the host: rank 1 raises before the collective and leaves; rank 0 must
    get an error from the handshake (short process-group timeout), not hang."""
    from igs_b200 import dist as idist

    try:
        _init(rank, world, port, "gloo", timeout_s=8)
        if rank == 1:
            raise RuntimeError("injected failure before the collective")
        idist.check_consistent((1, 3, 8, 8))
        q.put((rank, "no error"))
    except Exception as exc:  # noqa: BLE001
        q.put((rank, type(exc).__name__))


def test_dead_peer_gives_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_peer_dies, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()
    assert res[1] == "RuntimeError" and res[0] != "no error", res


def _fit_target(H, W):
    yy, xx = torch.meshgrid(torch.linspace(-1, 1, H), torch.linspace(-1, 1, W), indexing="ij")
    return torch.stack([0.5 + 0.4 * torch.sin(3 * xx + c) * torch.cos(2 * yy - c) for c in range(3)])[None]


def _spread(model):
    """Makes the start anisotropic and rotated (a function of each gaussian's own position, so
    every split of the gaussians gets the same values).  With the fitter's isotropic start the
    rotation gradient is rounding noise, which Adam's normalisation would turn into steps of
    the size of the learning rate with a sign that depends on the summation order."""
    with torch.no_grad():
        model.log_scale.add_(0.4 * torch.sin(5.0 * model.position))
        model.rotation.add_(2.0 * model.position[..., 0] - model.position[..., 1])


def _worker_sharded_fit(rank, world, port, backend, q):
    """Three Adam steps of the gaussian-sharded per-image fit: the loss of every step and the
    parameters of all ranks afterwards."""
    from igs_b200 import fit

    try:
        _init(rank, world, port, backend)
        dev = torch.device("cuda", rank) if backend == "nccl" else torch.device("cpu")
        tgt = _fit_target(18, 22).to(dev)
        model = fit.ShardedImageFitter(53, channels=3, image=tgt.cpu(), init_log_scale=-1.5,
                                       backend=None if backend == "nccl" else OracleBackend).to(dev)
        _spread(model)
        if backend == "nccl":
            # through the package's own loop (which keeps a sharded model out of graph capture)
            losses = fit.fit(model, tgt, steps=3, lr=2e-2, graph=True).tolist()
        else:
            opt = torch.optim.Adam(model.parameters(), lr=2e-2)
            losses = []
            for _ in range(3):
                opt.zero_grad(set_to_none=True)
                loss = torch.nn.functional.mse_loss(model((18, 22)), tgt)
                loss.backward()
                opt.step()
                losses.append(float(loss.detach()))
        full = {k: v.cpu().numpy() for k, v in model.gathered().items()}
        q.put((rank, model.range, losses, full, None))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # noqa: BLE001 - reported to the parent
        q.put((rank, None, None, None, repr(exc)))


def _run_sharded_fit(world, backend):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_sharded_fit, args=(r, world, port, backend, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for r in res:
        assert r[4] is None, f"rank {r[0]} failed: {r[4]}"
    return sorted(res, key=lambda r: r[0])


def _check_sharded_fit(two, one, tol):
    (_, rng1, losses1, full1, _), = one
    assert rng1 == (0, 53) and [r[1] for r in two] == [(0, 27), (27, 53)]
    for r in two:
        assert np.allclose(r[2], losses1, rtol=tol, atol=0), (r[2], losses1)
        for k, v in r[3].items():
            assert v.shape == full1[k].shape
            assert_close(v, full1[k], tol, f"{k} after 3 steps, seen from rank {r[0]}")
    assert losses1[2] < losses1[0]


def test_sharded_image_fitter_two_ranks_equal_one_gloo():
    """The fit over two ranks walks the same path as over one: per-step loss and, after three
    Adam steps, every parameter (gathered) agree."""
    _check_sharded_fit(_run_sharded_fit(2, "gloo"), _run_sharded_fit(1, "gloo"), 1e-5)


@pytest.mark.gpu
def test_sharded_image_fitter_on_one_gpu_follows_the_plain_fitter():
    """A process group of one rank: the sharded fitter (sums, all-reduce, normalise) against
    ImageFitter through autograd, same three Adam steps."""
    from igs_b200 import fit

    (_, rng, losses, full, _), = _run_sharded_fit(1, "nccl")
    dev = torch.device("cuda", 0)
    tgt = _fit_target(18, 22).to(dev)
    model = fit.ImageFitter(53, channels=3, image=tgt.cpu(), init_log_scale=-1.5).to(dev)
    _spread(model)
    opt = torch.optim.Adam(model.parameters(), lr=2e-2)
    plain = []
    for _ in range(3):
        opt.zero_grad(set_to_none=True)
        loss = torch.nn.functional.mse_loss(model((18, 22)), tgt)
        loss.backward()
        opt.step()
        plain.append(float(loss.detach()))
    assert rng == (0, 53)
    assert np.allclose(losses, plain, rtol=1e-4, atol=0), (losses, plain)
    for k, v in full.items():
        assert_close(v, getattr(model, k).detach().cpu().numpy(), 1e-4, f"{k} after 3 steps")


@pytest.mark.gpu
def test_sharded_image_fitter_two_gpus_nccl():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    _check_sharded_fit(_run_sharded_fit(2, "nccl"), _run_sharded_fit(1, "nccl"), 1e-4)


@pytest.mark.gpu
def test_gaussian_sharded_two_gpus_nccl():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    _check_against_single(_run_sharded(2, "nccl"))
