"""The sharded population step on two GPUs: both exchanges go through the library's own
communicator (hses_comm_* behind the C ABI); the ranks must finish a step with bit-identical
parameters, and those must match the single-GPU step within 1e-3.  Needs two CUDA devices
(skipped otherwise); the ranks are child processes, one per GPU."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DIMS, T, BM, RANK, SIGMA = [784, 128, 128, 10], 8, 1, 64, 0.02


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(n_pop):
    g = np.random.Generator(np.random.PCG64(0))
    img = g.random((n_pop * BM, 784), dtype=np.float32)
    img[g.random((n_pop * BM, 784)) < 0.8] = 0.0
    return img, g.integers(0, 10, n_pop * BM).astype(np.int32)


def _make_step(dev, lo, n_local, n_total, solver):
    from hyperscalees_b200 import models, noiser
    net = models.SnnMlp(DIMS, tau_m=20.0, v_th=0.3, seed=0, device=dev)
    frozen, nz = noiser.init_noiser(net.params(), SIGMA, 0.01, 0, False, 0, RANK, solver)
    keys = models.default_base_keys(len(DIMS))
    return models.PopulationStep(net, frozen, nz, keys, T, n_local, BM, first_thread=lo, cache="auto",
                                 n_total=n_total if n_local == n_total else None)


def _checksum(params):
    # sum of the bit patterns: equal sums over equal-length vectors of identical bits
    return [int(p.view(torch.int32).to(torch.int64).sum().item()) for p in params]


def _rank_main(rank, world, port, n_pop, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from hyperscalees_b200 import core, noiser, parallel
    ctx = core.get_context(rank)
    comm = parallel.Comm.from_process_group(ctx)
    img, labels = _inputs(n_pop)
    lo, hi = parallel.shard_range(n_pop, rank, world)
    di, dl = torch.as_tensor(img[lo * BM:hi * BM], device=dev), torch.as_tensor(labels[lo * BM:hi * BM], device=dev)
    step = _make_step(dev, lo, hi - lo, n_pop, noiser.Solver.adamw(0.01))
    sums, fits = [], []
    for it in range(2):
        raw = step.eval(di, dl, [1, 2, 3, 4])   # the Poisson stream is indexed inside the call's batch
        full = parallel.allgather_fitness(raw, n_pop, comm=comm)
        fits.append(full.cpu().numpy())
        step.update_sharded(full, comm=comm)
        torch.cuda.synchronize()
        comm.async_error()
        sums.append(_checksum(step.params))
    status = ctx.device_status()
    params = [p.cpu().numpy() for p in step.params]
    comm.destroy()
    dist.destroy_process_group()
    q.put((rank, sums, fits[0], params if rank == 0 else None, status))


def test_two_gpu_step_identical_parameters_and_single_gpu_parity(hs):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import torch.multiprocessing as mp
    from hyperscalees_b200 import noiser, parallel
    n_pop, world = 4096, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, n_pop, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted((q.get(timeout=600) for _ in procs), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=120)
    assert all(r[4] == 0 for r in res), "a kernel gave up on a bounded wait"
    # every rank ends every step with the same bits in every parameter
    assert res[0][1] == res[1][1]
    assert np.array_equal(res[0][2], res[1][2])
    # the same two steps on one GPU: each rank's Poisson stream is indexed inside its own batch, so
    # the single-GPU run evaluates the two shards as two calls, then updates once with the whole vector
    dev = torch.device("cuda", 0)
    img, labels = _inputs(n_pop)
    whole = _make_step(dev, 0, n_pop, n_pop, noiser.Solver.adamw(0.01))
    whole.build_caches(0, n_pop)
    shards = []
    for r in range(world):
        lo, hi = parallel.shard_range(n_pop, r, world)
        st = _make_step(dev, lo, hi - lo, n_pop, noiser.Solver.adamw(0.01))
        st.params = whole.params
        st.net.weights, st.net.out_gain = whole.params[:-1], whole.params[-1]
        shards.append((st, torch.as_tensor(img[lo * BM:hi * BM], device=dev),
                       torch.as_tensor(labels[lo * BM:hi * BM], device=dev)))
    for it in range(2):
        raw = torch.cat([st.eval(di, dl, [1, 2, 3, 4]) for st, di, dl in shards])
        if it == 0:
            assert np.array_equal(raw.cpu().numpy(), res[0][2])   # the forward is the same computation
        whole.update(raw)
    for got, want in zip(res[0][3], [p.cpu().numpy() for p in whole.params]):
        assert np.abs(got - want).max() <= 1e-3 * max(np.abs(want).max(), 1e-6)


def _peer_main(rank, world, port, n_pop, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from hyperscalees_b200 import core, parallel
    ctx = core.get_context(rank)
    comm = parallel.Comm.from_process_group(ctx)
    px = parallel.PeerExchange(n_pop, ctx)
    lo, hi = parallel.shard_range(n_pop, rank, world)
    same, statuses = [], []
    for step in range(5):
        g = torch.Generator(device=dev).manual_seed(100 * step + rank)
        local = torch.randn(hi - lo, device=dev, generator=g)
        got = px.exchange(local)
        want = parallel.allgather_fitness(local, n_pop, comm=comm)
        torch.cuda.synchronize()
        same.append(bool(torch.equal(got, want)))
    statuses.append(ctx.device_status())
    # a step in which rank 1 withholds its shard (the failure is made on the host: no kernel is asked to
    # misbehave): every wait runs out after about a second, says so in the status word, and returns
    sentinel = torch.full((n_pop,), -7.0, device=dev)
    local = torch.ones(hi - lo, device=dev)
    px.exchange(local, out=sentinel, publish=(rank != 1))
    torch.cuda.synchronize()
    statuses.append(ctx.device_status())
    untouched = bool((sentinel == -7.0).all().item())
    dist.barrier()
    # the next step works again
    got = px.exchange(local * (rank + 1))
    want = parallel.allgather_fitness(local * (rank + 1), n_pop, comm=comm)
    torch.cuda.synchronize()
    same.append(bool(torch.equal(got, want)))
    statuses.append(ctx.device_status())
    px.destroy()
    comm.destroy()
    dist.destroy_process_group()
    q.put((rank, same, statuses, untouched))


def test_peer_memory_fitness_exchange_and_its_bounded_wait(hs):
    """The peer-memory exchange returns the all-gather's bits; when a rank withholds its shard the
    other ranks' waits run out (bit 9 of the device status), the output is left alone, nothing
    hangs, and the next step works."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import torch.multiprocessing as mp
    n_pop, world = 4096, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_peer_main, args=(r, world, port, n_pop, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted((q.get(timeout=600) for _ in procs), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=120)
    for rank, same, statuses, untouched in res:
        assert all(same), f"rank {rank}: exchange differs from the all-gather"
        assert statuses[0] == 0 and statuses[2] == 0
        assert statuses[1] == 1 << 9, f"rank {rank}: the withheld shard was not noticed"
        assert untouched
