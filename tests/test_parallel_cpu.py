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


# ---------------------------------------------------------------------------------------------
# the communicator behind the C ABI, driven on the CPU through a stand-in for NCCL
# ---------------------------------------------------------------------------------------------
_COMM_SCRIPT = r"""
import os, sys
import torch
sys.path.insert(0, sys.argv[1])
from hyperscalees_b200 import parallel
mode = sys.argv[2]
uid = parallel.Comm.unique_id()
assert len(uid) == 128
if mode == "init_fails":
    try:
        parallel.Comm(uid, 0, 1)
    except parallel.CommError as e:
        assert "ncclCommInitRank failed" in str(e), str(e)
        print("ok")
    sys.exit(0)
try:
    parallel.Comm(uid, 3, 2)
except parallel.CommError as e:
    assert "rank must be in [0, world)" in str(e)
else:
    raise AssertionError("a rank outside the world must be refused")
comm = parallel.Comm(uid, 0, 2)
assert (comm.rank, comm.world) == (0, 2)
local = torch.arange(4, dtype=torch.float32)
if mode == "ok":
    out = comm.allgather_fitness(local, torch.empty(8))
    assert torch.equal(out, torch.cat([local, local]))
    g = torch.ones(5)
    comm.allreduce_grads(g)
    assert torch.equal(g, torch.full((5,), 2.0))
    comm.async_error()
    comm.destroy()
elif mode == "collective_fails":
    try:
        comm.allgather_fitness(local, torch.empty(8))
    except parallel.CommError as e:
        assert "ncclAllGather failed" in str(e)
    else:
        raise AssertionError("the failing all-gather must raise")
    # the communicator is now marked broken: nothing more is enqueued on it
    try:
        comm.allreduce_grads(torch.ones(3))
    except parallel.CommError as e:
        assert "error state" in str(e)
    else:
        raise AssertionError("a broken communicator must refuse further work")
    comm.destroy()   # aborts instead of waiting
elif mode == "peer_left":
    try:
        comm.async_error()
    except parallel.CommError as e:
        assert "remote process exited" in str(e)
    else:
        raise AssertionError("the reported remote error must raise")
    try:
        comm.allgather_fitness(local, torch.empty(8))
    except parallel.CommError:
        pass
    else:
        raise AssertionError("a broken communicator must refuse further work")
    comm.destroy()
print("ok")
"""


@pytest.fixture(scope="module")
def fake_nccl(tmp_path_factory):
    import subprocess
    d = tmp_path_factory.mktemp("fake_nccl")
    so = d / "libfake_nccl.so"
    src = os.path.join(os.path.dirname(os.path.abspath(__file__)), "support", "fake_nccl.c")
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", str(so), src], check=True)
    return so


@pytest.mark.parametrize("mode,env,last_call", [
    ("ok", {}, "ncclCommDestroy"),
    ("init_fails", {"FAKE_NCCL_FAIL": "init"}, "ncclCommInitRank"),
    ("collective_fails", {"FAKE_NCCL_FAIL": "allgather"}, "ncclCommAbort"),
    ("peer_left", {"FAKE_NCCL_ASYNC": "6"}, "ncclCommAbort"),
])
def test_comm_c_abi_against_a_stand_in_for_nccl(fake_nccl, tmp_path, mode, env, last_call):
    """hses_comm_* and the two collectives through ctypes, with NCCL replaced by a host stand-in
    whose calls can be made to fail: a failing call surfaces as CommError, marks the communicator
    broken, and the broken communicator is aborted, not destroyed."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    log = tmp_path / "calls.log"
    e = dict(os.environ, HSES_NCCL_LIBRARY=str(fake_nccl), FAKE_NCCL_LOG=str(log), **env)
    res = subprocess.run([sys.executable, "-c", _COMM_SCRIPT, root, mode], env=e, capture_output=True, text=True,
                         timeout=120)
    assert res.returncode == 0 and res.stdout.strip().endswith("ok"), res.stdout + res.stderr
    assert log.read_text().split()[-1] == last_call


# ---------------------------------------------------------------------------------------------
# host-side failure detection: a rank that leaves between steps, a rank that stops
# ---------------------------------------------------------------------------------------------
def _hb_worker(rank, world, path, behaviour, q):
    from hyperscalees_b200 import parallel
    store = dist.FileStore(path, world)
    hb = parallel.Heartbeat(store, rank, world, timeout=3.0)
    steps_done = 0
    try:
        for step in range(4):
            if rank == 1 and step == 2:
                if behaviour == "leaves":
                    hb.leave()          # between steps: nothing of this rank is in flight
                    break
                if behaviour == "stops":
                    break               # never announces step 2 and says nothing
            hb.enter(step)
            steps_done += 1
        q.put((rank, steps_done, None))
    except parallel.RankLeft as e:
        q.put((rank, steps_done, str(e)))


@pytest.mark.parametrize("behaviour,needle", [("leaves", "rank 1 left before step 2"),
                                              ("stops", "did not reach step 2"), ("healthy", None)])
def test_heartbeat_tells_the_others_before_their_next_launch(tmp_path, behaviour, needle):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    path = str(tmp_path / "store")
    procs = [ctx.Process(target=_hb_worker, args=(r, 2, path, behaviour, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict((r[0], r[1:]) for r in (q.get(timeout=120) for _ in procs))
    for p in procs:
        p.join(timeout=60)
    if needle is None:
        assert res[0] == (4, None) and res[1] == (4, None)
    else:
        assert res[0][0] == 2 and needle in res[0][1]     # rank 0 finished steps 0 and 1, then learned of it
        assert res[1] == (2, None)
