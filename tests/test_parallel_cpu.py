"""Host-side logic of the multi-GPU population step, exercised with two gloo ranks on the CPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def test_shard_ranges_are_pair_aligned_and_cover_the_population():
    from hyperscalees_b200 import parallel
    for n_pop, world in [(256, 1), (256, 2), (8192, 8), (30, 4), (65536, 8), (6, 4)]:
        prev = 0
        for r in range(world):
            lo, hi = parallel.shard_range(n_pop, r, world)
            assert lo == prev and lo % 2 == 0 and hi % 2 == 0 and hi >= lo
            prev = hi
        assert prev == n_pop
        sizes = parallel.shard_sizes(n_pop, world)
        assert max(sizes) - min(sizes) <= 2
    with pytest.raises(ValueError):
        parallel.shard_range(7, 0, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_pop, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from hyperscalees_b200 import parallel
    lo, hi = parallel.shard_range(n_pop, rank, world)
    full = torch.arange(n_pop, dtype=torch.float32) * 0.5 - 3.0   # what an unsharded run would hold
    got = parallel.allgather_fitness(full[lo:hi].clone(), n_pop)
    grads = [torch.full((2, 3), float(rank + 1))]
    parallel.allreduce_grads(grads)
    q.put((rank, torch.equal(got, full), grads[0][0, 0].item()))
    dist.destroy_process_group()


@pytest.mark.parametrize("n_pop", [16, 10])   # equal shards, and shards of unequal size
def test_fitness_allgather_two_ranks(n_pop):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n_pop, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert [r[1] for r in res] == [True, True]
    assert [r[2] for r in res] == [3.0, 3.0]
