"""Population sharding across the GPUs of one node.

The population step shards by contiguous, pair-aligned member ranges: rank g
owns thread ids [lo_g, hi_g) with lo_g even, so the two members of an
antithetic pair always sit on the same GPU.  Every rank regenerates its own
members' noise from (key, epoch, thread id) — the same rule as the reference's
multi-GPU script (llm_experiments/snn_mnist_train_multi_gpu.py:146-149,
186-205) — so the only exchange of a step is the all-gather of the raw fitness
vector (plus, for the sharded update, one sum of the flat gradient buffer);
afterwards every rank holds the full vector, normalises it identically and
applies the same update.

Two transports carry the two exchanges: `Comm`, the library's own communicator
behind the C ABI (hses_comm_* / hses_allgather_fitness / hses_allreduce_grads,
the calls a Rust trainer would make), and torch.distributed process groups
(NCCL on GPUs, gloo for the CPU tests of the host logic).  `Heartbeat` is the
host-side failure detection: ranks announce every step they enter in a key-value
store and learn, before their next launch, of a peer that left or stopped.
"""
from __future__ import annotations

import ctypes as C
import time
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(n_pop: int, rank: int, world: int) -> Tuple[int, int]:
    """Members [lo, hi) owned by `rank`: whole antithetic pairs, sizes differing by at most one pair."""
    if n_pop % 2 != 0:
        raise ValueError("the population must consist of whole antithetic pairs (n_pop even)")
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    pairs = n_pop // 2
    base, extra = divmod(pairs, world)
    lo_pair = rank * base + min(rank, extra)
    hi_pair = lo_pair + base + (1 if rank < extra else 0)
    return 2 * lo_pair, 2 * hi_pair


def shard_sizes(n_pop: int, world: int) -> List[int]:
    return [hi - lo for lo, hi in (shard_range(n_pop, r, world) for r in range(world))]


class CommError(RuntimeError):
    """A collective, its communicator or a peer failed; the communicator must be dropped."""


class Comm:
    """One rank's communicator behind the C ABI.  Rank 0 creates the id (`Comm.unique_id()`) and
    hands it to the others out of band (`Comm.from_process_group` does it through
    torch.distributed); the device of the calling thread must be the rank's GPU."""

    def __init__(self, unique_id: bytes, rank: int, world: int, ctx=None):
        from . import _lib
        self._lib, self.L = _lib, _lib.load()
        if len(unique_id) != 128:
            raise ValueError("the communicator id is 128 bytes long")
        self.rank, self.world = rank, world
        handle = C.c_void_p()
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        self._check(self.L.hses_comm_init(ctx.handle if ctx is not None else None, buf, rank, world,
                                          C.byref(handle)))
        self.handle = handle

    @staticmethod
    def unique_id() -> bytes:
        from . import _lib
        L = _lib.load()
        buf = (C.c_uint8 * 128)()
        st = L.hses_comm_unique_id(buf)
        if st != 0:
            raise CommError(L.hses_last_error().decode())
        return bytes(buf)

    @classmethod
    def from_process_group(cls, ctx=None, group: Optional[dist.ProcessGroup] = None) -> "Comm":
        """Builds the communicator of every rank of an initialised torch.distributed group: rank
        0's id travels as one broadcast."""
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        box = [cls.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0, group=group)
        return cls(box[0], rank, world, ctx)

    def _check(self, status: int) -> None:
        if status != 0:
            raise CommError(f"hses status {status}: {self.L.hses_last_error().decode()}")

    @staticmethod
    def _stream(t: torch.Tensor) -> int:
        # host tensors only reach here with a stand-in for NCCL (the CPU tests of this wrapper)
        from .core import current_stream
        return current_stream(t.device) if t.is_cuda else 0

    def async_error(self) -> None:
        """Raises CommError once NCCL has reported a failed collective on this communicator."""
        self._check(self.L.hses_comm_async_error(self.handle))

    def allgather_fitness(self, local: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        self._check(self.L.hses_allgather_fitness(self.handle, self._stream(local), local.data_ptr(), local.numel(),
                                                  out.data_ptr()))
        return out

    def allreduce_grads(self, grads: torch.Tensor) -> torch.Tensor:
        self._check(self.L.hses_allreduce_grads(self.handle, self._stream(grads), grads.data_ptr(), grads.numel()))
        return grads

    def destroy(self, abort: bool = False) -> None:
        if self.handle is not None:
            h, self.handle = self.handle, None
            st = self.L.hses_comm_abort(h) if abort else self.L.hses_comm_destroy(h)
            if st != 0 and not abort:
                raise CommError(self.L.hses_last_error().decode())


def _world(group, comm) -> Tuple[int, int]:
    if comm is not None:
        return comm.rank, comm.world
    if dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def allgather_fitness(local: torch.Tensor, n_pop: int, group: Optional[dist.ProcessGroup] = None,
                      comm: Optional[Comm] = None) -> torch.Tensor:
    """All-gather the per-member raw fitness of every shard into the full (n_pop,) vector, in
    thread-id order, through `comm` when given, else through torch.distributed (NCCL with CUDA
    tensors, gloo with CPU tensors)."""
    rank, world = _world(group, comm)
    if world == 1:
        if local.numel() != n_pop:
            raise ValueError("single-rank fitness vector must cover the whole population")
        return local
    sizes = shard_sizes(n_pop, world)
    if local.numel() != sizes[rank]:
        raise ValueError(f"rank {rank} owns {sizes[rank]} members but passed {local.numel()} fitness values")

    def gather(dst, src):
        if comm is not None:
            comm.allgather_fitness(src, dst)
        else:
            dist.all_gather_into_tensor(dst, src, group=group)

    if len(set(sizes)) == 1:
        out = torch.empty(n_pop, dtype=local.dtype, device=local.device)
        gather(out, local.contiguous())
        return out
    # shards of unequal size: pad every shard to the largest one, gather, drop the padding
    m = max(sizes)
    padded = torch.zeros(m, dtype=local.dtype, device=local.device)
    padded[:local.numel()] = local
    out = torch.empty(world * m, dtype=local.dtype, device=local.device)
    gather(out, padded)
    return torch.cat([out[r * m:r * m + sizes[r]] for r in range(world)])


def allreduce_grads(grads, group: Optional[dist.ProcessGroup] = None, comm: Optional[Comm] = None) -> None:
    """Second exchange of the sharded update: sum the partial gradients computed per shard (each
    rank called the update with its own first_thread and n_total = n_pop).  `grads` is the flat
    buffer of hses_population_grads or a list of tensors.  An all-reduce hands every rank the same
    bits (whatever order the library summed in), so ranks that start a step with identical
    parameters end it with identical parameters; the sum's order, and with it the last bits,
    may differ from the single-GPU contraction (the tests hold the two to 1e-3 relative)."""
    _, world = _world(group, comm)
    if world == 1:
        return
    for g in (grads if isinstance(grads, (list, tuple)) else [grads]):
        if comm is not None:
            comm.allreduce_grads(g)
        else:
            dist.all_reduce(g, op=dist.ReduceOp.SUM, group=group)


class PeerExchange:
    """The fitness exchange over peer memory instead of a collective (hses_fitness_publish /
    hses_fitness_wait): every rank's kernel stores its shard into every rank's window over NVLink and
    raises a flag; a bounded wait kernel collects the vector.  The windows are shared through CUDA
    IPC handles, which travel through torch.distributed (any backend).  All ranks of one node."""

    def __init__(self, n_pop: int, ctx=None, group: Optional[dist.ProcessGroup] = None):
        import ctypes as C
        from . import _lib, core
        self.ctx = ctx if ctx is not None else core.get_context()
        self.lib = _lib.load()
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.n_pop = n_pop
        self.tag = 0
        own = C.c_void_p()
        handle = (C.c_uint8 * 64)()
        _lib.check(self.lib.hses_peer_alloc(self.ctx.handle, n_pop, C.byref(own), handle))
        self.own = own.value
        handles: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.windows = (C.c_void_p * self.world)()
        self.opened = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.windows[r] = self.own
                continue
            w = C.c_void_p()
            buf = (C.c_uint8 * 64).from_buffer_copy(h)
            _lib.check(self.lib.hses_peer_open(self.ctx.handle, buf, C.byref(w)))
            self.windows[r] = w.value
            self.opened.append(w.value)
        dist.barrier(group=group)   # every window is mapped everywhere before the first store

    def exchange(self, local: torch.Tensor, out: Optional[torch.Tensor] = None, publish: bool = True) -> torch.Tensor:
        """local: this rank's shard (shard_range order).  Returns the (n_pop,) vector once all shards of this
        step have arrived; when one does not, the context's device status carries bit 9 and the result is
        not valid.  publish=False withholds this rank's shard (tests of the bounded wait)."""
        from . import _lib
        from .core import current_stream
        lo, hi = shard_range(self.n_pop, self.rank, self.world)
        if local.numel() != hi - lo or local.dtype != torch.float32 or not local.is_contiguous():
            raise ValueError("local must be this rank's contiguous f32 shard")
        if out is None:
            out = torch.empty(self.n_pop, dtype=torch.float32, device=local.device)
        self.tag += 1
        st = current_stream()
        if publish:   # the usual step: one launch stores this rank's shard everywhere and waits for the others'
            _lib.check(self.lib.hses_fitness_exchange(self.ctx.handle, st, local.data_ptr(), hi - lo, lo, self.n_pop,
                                                      self.windows, self.rank, self.world, self.tag, out.data_ptr()))
        else:
            _lib.check(self.lib.hses_fitness_wait(self.ctx.handle, st, self.own, self.n_pop, self.world, self.tag,
                                                  out.data_ptr()))
        return out

    def destroy(self) -> None:
        """Unmaps the peers' windows and frees this rank's.  Call it on every rank, with no exchange in flight."""
        from . import _lib
        torch.cuda.synchronize()
        for w in self.opened:
            _lib.check(self.lib.hses_peer_close(w))
        self.opened = []
        if dist.is_initialized():
            dist.barrier()   # nobody frees a window that a peer still has mapped and may write
        if self.own:
            _lib.check(self.lib.hses_peer_free(self.own))
            self.own = None


class RankLeft(CommError):
    """A peer announced that it left, or stopped announcing steps."""


class Heartbeat:
    """Host-side failure detection for the sharded step, over any key-value store with
    set/get/add (torch.distributed's TCPStore / FileStore / HashStore).  Every rank calls
    `enter(step)` before it launches a step: the call publishes the step, then waits until every
    peer has published the same step or has said goodbye; a peer that left (`leave()`), or one
    that does not arrive within `timeout` seconds, raises RankLeft on the others BEFORE they
    enqueue a collective that could never finish.  A rank leaves only between steps."""

    def __init__(self, store, rank: int, world: int, timeout: float = 30.0, poll: float = 0.01, prefix: str = "hb"):
        self.store, self.rank, self.world, self.timeout, self.poll, self.prefix = store, rank, world, timeout, poll, prefix
        self.store.set(self._key("left", rank), "0")
        self.store.set(self._key("step", rank), "-1")

    def _key(self, what: str, rank: int) -> str:
        return f"{self.prefix}/{what}/{rank}"

    def _read(self, what: str, rank: int, default: int) -> int:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(what, rank)]):
                return default
            return int(bytes(self.store.get(self._key(what, rank))).decode())
        except (RuntimeError, ValueError, KeyError):
            return default

    def leave(self) -> None:
        self.store.set(self._key("left", self.rank), "1")

    def enter(self, step: int) -> None:
        self.store.set(self._key("step", self.rank), str(step))
        deadline = time.monotonic() + self.timeout
        pending = [r for r in range(self.world) if r != self.rank]
        while pending:
            still = []
            for r in pending:
                # a peer that has published this step takes part in it, whatever it says afterwards:
                # a rank leaves only between steps, so its goodbye concerns the next one
                if self._read("step", r, -1) >= step:
                    continue
                if self._read("left", r, 0) == 1:
                    raise RankLeft(f"rank {r} left before step {step}")
                still.append(r)
            pending = still
            if pending:
                if time.monotonic() > deadline:
                    raise RankLeft(f"rank(s) {pending} did not reach step {step} within {self.timeout} s")
                time.sleep(self.poll)
