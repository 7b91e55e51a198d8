"""Tensor-level wrappers over the C ABI: every function checks its torch
tensors (CUDA, fp32, unit inner stride), forwards raw pointers, shapes and row
strides, and enqueues on torch's current stream.  PyTorch only supplies device
memory and streams here; all arithmetic happens in the CUDA library.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Sequence, Tuple

import torch

from . import _lib
from .core import current_stream, get_context

RESET_HARD, RESET_SUBTRACT = 0, 1
REWARD_LOGLIK, REWARD_BINARY = 0, 1
SGD, ADAM, ADAMW = 0, 1, 2
LAYOUT_NAR, LAYOUT_NRA = 0, 1
ALGO_AUTO, ALGO_SIMT, ALGO_TENSOR, ALGO_PAIR = 0, 1, 2, 3

_U64 = (1 << 64) - 1


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _check(t: torch.Tensor, name: str, dtype=torch.float32, ndim: Optional[int] = None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise ValueError(f"{name} must have {ndim} dims, got {t.dim()}")
    if t.dim() > 0 and t.stride(-1) != 1 and t.size(-1) > 1:
        raise ValueError(f"{name} must have unit stride along its last dim")


def _rows_2d(t: torch.Tensor, name: str) -> Tuple[int, int, int]:
    """View a (..., cols) tensor whose leading dims are mutually contiguous as
    pitched rows; returns (rows, cols, row_stride)."""
    cols = t.size(-1)
    rows = t.numel() // max(cols, 1)
    stride = t.stride(-2) if t.dim() >= 2 else cols
    expect = stride
    for d in range(t.dim() - 2, -1, -1):
        if t.size(d) != 1 and t.stride(d) != expect:
            raise ValueError(f"{name}: leading dims must be contiguous over pitched rows")
        expect *= t.size(d)
    return rows, cols, stride


def noise_seed(key: int, true_epoch: int, true_thread: int) -> int:
    return int(_lib.load().hses_noise_seed(C.c_uint64(key & _U64), true_epoch, true_thread))


def normal_fill(seed: int, n: int, device=None) -> torch.Tensor:
    ctx = get_context(device)
    out = torch.empty(n, dtype=torch.float32, device=torch.device("cuda", ctx.device))
    _lib.check(_lib.load().hses_normal_fill(ctx.handle, current_stream(), C.c_uint64(seed & _U64),
                                            _ptr(out), n))
    return out


def lora_factors(key: int, epoch: int, noise_reuse: int, rank: int, a: int, b: int,
                 base_sigma: float, n_members: int, first_thread: int = 0,
                 thread_ids: Optional[torch.Tensor] = None, layout: int = LAYOUT_NAR,
                 want_a: bool = True, want_b: bool = True, device=None):
    ctx = get_context(device)
    dev = torch.device("cuda", ctx.device)
    if thread_ids is not None:
        _check(thread_ids, "thread_ids", torch.int32, 1)
        n_members = thread_ids.numel()
    sa = (n_members, a, rank) if layout == LAYOUT_NAR else (n_members, rank, a)
    sb = (n_members, b, rank) if layout == LAYOUT_NAR else (n_members, rank, b)
    A = torch.empty(sa, dtype=torch.float32, device=dev) if want_a else None
    B = torch.empty(sb, dtype=torch.float32, device=dev) if want_b else None
    _lib.check(_lib.load().hses_lora_factors(
        ctx.handle, current_stream(), C.c_uint64(key & _U64), epoch, noise_reuse, _ptr(thread_ids),
        first_thread, n_members, rank, a, b, base_sigma, layout, _ptr(A), _ptr(B)))
    return A, B


def dense_noise(key: int, epoch: int, noise_reuse: int, rows: int, cols: int, base_sigma: float,
                n_members: int, first_thread: int = 0, thread_ids: Optional[torch.Tensor] = None,
                device=None) -> torch.Tensor:
    ctx = get_context(device)
    if thread_ids is not None:
        _check(thread_ids, "thread_ids", torch.int32, 1)
        n_members = thread_ids.numel()
    out = torch.empty((n_members, rows, cols), dtype=torch.float32,
                      device=torch.device("cuda", ctx.device))
    _lib.check(_lib.load().hses_dense_noise(
        ctx.handle, current_stream(), C.c_uint64(key & _U64), epoch, noise_reuse, _ptr(thread_ids),
        first_thread, n_members, rows, cols, base_sigma, _ptr(out)))
    return out


def poisson_encode(probs: torch.Tensor, T: int, seeds: Sequence[int],
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """probs (batch, in_dim) pitched -> spikes (T, batch, in_dim) with the same pitch."""
    _check(probs, "probs", ndim=2)
    batch, in_dim = probs.shape
    stride = probs.stride(0) if batch > 1 else max(probs.stride(0), in_dim)
    if out is None:
        buf = torch.empty((T, batch, stride), dtype=torch.float32, device=probs.device)
        out = buf[:, :, :in_dim]
    else:
        _check(out, "out", ndim=3)
        if tuple(out.shape) != (T, batch, in_dim) or out.stride(1) != stride or \
                (T > 1 and out.stride(0) != batch * stride):
            raise ValueError("out must be (T, batch, in_dim) with the pitch of probs")
    ctx = get_context(probs.device)
    sd = (C.c_uint32 * 4)(*[int(s) & 0xFFFFFFFF for s in seeds])
    _lib.check(_lib.load().hses_poisson_encode(ctx.handle, current_stream(), _ptr(probs), batch,
                                               in_dim, stride, T, sd, _ptr(out)))
    return out


def prng_normal_half(total_threads: int, mean: float, std: float, seeds: Sequence[int], device=None,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """total_threads * 128 normals of the hybrid Tausworthe stream (reference thread t fills
    out[128t, 128t+128))."""
    ctx = get_context(device)
    n = total_threads * 128
    if out is None:
        out = torch.empty(n, dtype=torch.float32, device=torch.device("cuda", ctx.device))
    else:
        _check(out, "out", ndim=1)
        if out.numel() != n:
            raise ValueError("out must hold total_threads * 128 values")
    sd = (C.c_uint32 * 4)(*[int(s) & 0xFFFFFFFF for s in seeds])
    _lib.check(_lib.load().hses_prng_normal_half(ctx.handle, current_stream(), _ptr(out), total_threads,
                                                 mean, std, sd))
    return out


def lif_scan(cur: torch.Tensor, tau_m: float, v_th: float, v: Optional[torch.Tensor] = None,
             reset_mode: int = RESET_HARD, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """cur (T, n, h) pitched -> spikes of the same layout; v (n, h) is updated in place."""
    _check(cur, "cur", ndim=3)
    T, n, h = cur.shape
    stride = cur.stride(1)
    if T > 1 and cur.stride(0) != n * stride:
        raise ValueError("cur: time steps must be n*row_stride apart")
    if out is None:
        buf = torch.empty((T, n, stride), dtype=torch.float32, device=cur.device)
        out = buf[:, :, :h]
    else:
        _check(out, "out", ndim=3)
        if tuple(out.shape) != (T, n, h) or out.stride(1) != stride:
            raise ValueError("out must match cur's shape and pitch")
    if v is not None:
        _check(v, "v", ndim=2)
        if tuple(v.shape) != (n, h) or (n > 1 and v.stride(0) != stride):
            raise ValueError("v must be (n, h) with cur's row pitch")
    ctx = get_context(cur.device)
    _lib.check(_lib.load().hses_lif_scan(ctx.handle, current_stream(), _ptr(cur), T, n, h, stride,
                                         _ptr(v), tau_m, v_th, reset_mode, _ptr(out)))
    return out


_workspaces = {}


def _workspace(device: torch.device, nbytes: int) -> Optional[torch.Tensor]:
    """Grow-only scratch buffer per (device, current stream): the library itself never allocates
    scratch, and calls on different streams must not share one.  A buffer that is outgrown is
    handed back to the allocator tied to the stream whose kernels may still be using it."""
    if nbytes == 0:
        return None
    stream = torch.cuda.current_stream(device)
    slot = (device, stream.cuda_stream)
    buf = _workspaces.get(slot)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            buf.record_stream(stream)
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _workspaces[slot] = buf
    return buf


def perturbed_linear(x: torch.Tensor, param: torch.Tensor, *, n_pop: int, bm: int, t_steps: int = 1,
                     sigma: float = 0.0, rank: int = 1, key: int = 0, epoch: int = 0,
                     first_thread: int = 0, noise_reuse: int = 0, perturb: bool = True,
                     lif: bool = False, tau_m: float = 20.0, v_th: float = 0.3,
                     reset_mode: int = RESET_HARD, out_scale: float = 1.0,
                     out: Optional[torch.Tensor] = None, want_potentials: bool = False,
                     algo: int = ALGO_AUTO, cache: Optional["FactorCache"] = None, precision: int = 0,
                     tmm: bool = False, x_half: Optional[torch.Tensor] = None,
                     out_half: Optional[torch.Tensor] = None, reuse_x_split: bool = False, n_groups: int = 1,
                     x_relu_square: bool = False):
    """do_mm over a population (+ optional LIF step).  x: (..., k) with
    t_steps*n_pop*bm rows; param: (a, k).  Returns out (rows, a) and, if asked,
    the charged potentials.  With `cache` the factors are read from it instead of
    being regenerated (same bits).  x_half: x once more as dense fp16 (rows, k) when it is exact
    there; out_half: a dense fp16 (rows, a) tensor that receives the spikes as well (lif only).
    x_relu_square: the layer's input is relu(x)^2; applied where the tensor-core path's prepass reads x, or, for
    calls that path does not take this way, by one pass of its own before the call.
    n_groups: `param` stacks that many parameters of equal shape along its rows, each with its own noise;
    `cache` must then be a GroupedFactorCache over them and `key` its key (tensor-core path only).
    reuse_x_split: the previous call on this device and stream had the same x and the same shapes
    (another projection of the same activation): its operand split of x is taken as it stands."""
    _check(x, "x")
    _check(param, "param", ndim=2)
    rows, k, xs = _rows_2d(x, "x")
    if rows != t_steps * n_pop * bm:
        raise ValueError(f"x has {rows} rows, expected t_steps*n_pop*bm = {t_steps * n_pop * bm}")
    a, k2 = param.shape
    if k2 != k:
        raise ValueError("param must be (a, k) with k = x's last dim")
    if out is None:
        out = torch.empty((rows, a), dtype=torch.float32, device=x.device)
    else:
        _check(out, "out", ndim=2)
        if tuple(out.shape) != (rows, a):
            raise ValueError("out must be (rows, a)")
    pot = None
    if want_potentials:
        pot = torch.empty((rows, out.stride(0)), dtype=torch.float32, device=x.device)[:, :a]
    g = _lib.LinearArgs()
    g.x, g.t_steps, g.n_pop, g.bm, g.k, g.x_row_stride = x.data_ptr(), t_steps, n_pop, bm, k, xs
    g.param, g.a, g.param_row_stride = param.data_ptr(), a, param.stride(0) if a > 1 else max(param.stride(0), k)
    g.sigma, g.rank, g.key, g.epoch = sigma, rank, key & _U64, epoch
    g.first_thread, g.noise_reuse, g.perturb, g.lif = first_thread, noise_reuse, int(perturb), int(lif)
    g.tau_m, g.v_th, g.reset_mode, g.out_scale = tau_m, v_th, reset_mode, out_scale
    g.out, g.out_row_stride = out.data_ptr(), out.stride(0) if rows > 1 else max(out.stride(0), a)
    g.potentials = pot.data_ptr() if pot is not None else None
    g.algo = algo
    g.precision = precision
    g.factor_order = int(tmm)   # do_Tmm: param is the reference's (in, out) matrix transposed
    g.x_split_valid = int(reuse_x_split)
    g.n_groups = int(n_groups)
    g.x_op = 1 if x_relu_square else 0
    if x_half is not None:
        if x_half.dtype != torch.float16 or not x_half.is_contiguous() or x_half.numel() != rows * k:
            raise ValueError("x_half must be a contiguous fp16 tensor of rows*k values")
        g.x_half = x_half.data_ptr()
    if out_half is not None:
        if out_half.dtype != torch.float16 or not out_half.is_contiguous() or out_half.numel() != rows * a:
            raise ValueError("out_half must be a contiguous fp16 tensor of rows*a values")
        g.out_half = out_half.data_ptr()
    if cache is not None:
        g.cache = C.pointer(cache.desc)
    L = _lib.load()
    need = int(L.hses_perturbed_linear_workspace_bytes(C.byref(g)))
    if g.x_op and need == 0:
        # not a call whose prepass applies the activation on the fly (0: the tensor-core path, which always
        # needs scratch, does not take it): one pass of its own, then the plain call
        xa = relu_square(x.reshape(rows, k) if x.is_contiguous() else x.contiguous().reshape(rows, k))
        g.x, g.x_row_stride, g.x_op = xa.data_ptr(), k, 0
        need = int(L.hses_perturbed_linear_workspace_bytes(C.byref(g)))
    ws = _workspace(x.device, need)
    g.workspace = ws.data_ptr() if ws is not None else None
    g.workspace_bytes = need
    ctx = get_context(x.device)
    _lib.check(L.hses_perturbed_linear(ctx.handle, current_stream(), C.byref(g)))
    return (out, pot) if want_potentials else out


def time_mean(x: torch.Tensor) -> torch.Tensor:
    """x (T, n, h) pitched -> dense (n, h) mean over T."""
    _check(x, "x", ndim=3)
    T, n, h = x.shape
    stride = x.stride(1)
    if T > 1 and x.stride(0) != n * stride:
        raise ValueError("x: time steps must be n*row_stride apart")
    out = torch.empty((n, h), dtype=torch.float32, device=x.device)
    ctx = get_context(x.device)
    _lib.check(_lib.load().hses_time_mean(ctx.handle, current_stream(), _ptr(x), T, n, h, stride,
                                          _ptr(out), h))
    return out


def fitness(logits: torch.Tensor, labels: torch.Tensor, reward: int = REWARD_LOGLIK) -> torch.Tensor:
    _check(logits, "logits", ndim=2)
    _check(labels, "labels", torch.int32, 1)
    logits = logits.contiguous()
    n, c = logits.shape
    out = torch.empty(n, dtype=torch.float32, device=logits.device)
    ctx = get_context(logits.device)
    _lib.check(_lib.load().hses_fitness(ctx.handle, current_stream(), _ptr(logits), n, c,
                                        _ptr(labels), reward, _ptr(out)))
    return out


def member_mean(per_sample: torch.Tensor, n_pop: int, bm: int) -> torch.Tensor:
    _check(per_sample, "per_sample", ndim=1)
    out = torch.empty(n_pop, dtype=torch.float32, device=per_sample.device)
    ctx = get_context(per_sample.device)
    _lib.check(_lib.load().hses_member_mean(ctx.handle, current_stream(), _ptr(per_sample), n_pop,
                                            bm, _ptr(out)))
    return out


def convert_fitnesses(raw: torch.Tensor, group_size: int = 0, want_stats: bool = False):
    _check(raw, "raw", ndim=1)
    out = torch.empty_like(raw)
    stats = torch.empty(2, dtype=torch.float32, device=raw.device) if want_stats else None
    ctx = get_context(raw.device)
    _lib.check(_lib.load().hses_convert_fitnesses(ctx.handle, current_stream(), _ptr(raw),
                                                  raw.numel(), group_size, _ptr(out), _ptr(stats)))
    return (out, stats) if want_stats else out


UPDATE_GRAD, UPDATE_RAW_ACC = 0, 1
PRECISION_FP32, PRECISION_BF16 = 0, 1


class FactorCache:
    """Raw factors of a range of antithetic pairs of one parameter, resident on the device
    (LoraNoiseCache, eggroll.rs:229-309).  Valid for the epoch bucket it was built for."""

    def __init__(self, key: int, epoch: int, noise_reuse: int, rank: int, a: int, b: int,
                 n_pairs: int, first_pair: int = 0, device=None):
        ctx = get_context(device)
        dev = torch.device("cuda", ctx.device)
        L = _lib.load()
        need = int(L.hses_factor_cache_bytes(n_pairs, rank, a, b))
        if need == 0:
            raise ValueError("empty factor cache")
        self.data = torch.empty(need // 4, dtype=torch.float32, device=dev)
        self.desc = _lib.FactorCacheDesc()
        with torch.cuda.device(dev):
            _lib.check(L.hses_factor_cache_build(ctx.handle, current_stream(), C.c_uint64(key & _U64),
                                                 epoch, noise_reuse, first_pair, n_pairs, rank, a, b,
                                                 _ptr(self.data), C.byref(self.desc)))
        self.n_pairs, self.rank, self.a, self.b = n_pairs, rank, a, b

    @property
    def A(self) -> torch.Tensor:
        """(n_pairs, a, rank) raw normals."""
        return self.data[: self.n_pairs * self.a * self.rank].view(self.n_pairs, self.a, self.rank)

    @property
    def B(self) -> torch.Tensor:
        """(n_pairs, b, rank) raw normals."""
        return self.data[self.n_pairs * self.a * self.rank:].view(self.n_pairs, self.b, self.rank)


class GroupedFactorCache:
    """The factors of several parameters of one shape (a_g, b) in the layout a grouped perturbed_linear
    call reads: A (n_pairs, G * a_g, rank) with the parameters' A blocks stacked like the parameters, then
    B (n_pairs, G, b, rank).  Assembled on the device from one FactorCache per parameter; the descriptor
    carries the first parameter's key, which the call passes as `key`."""

    def __init__(self, caches: Sequence["FactorCache"]):
        c0 = caches[0]
        for c in caches:
            if (c.n_pairs, c.rank, c.a, c.b) != (c0.n_pairs, c0.rank, c0.a, c0.b) or \
                    (c.desc.true_epoch, c.desc.first_pair) != (c0.desc.true_epoch, c0.desc.first_pair):
                raise ValueError("grouped caches must share shape, pairs and epoch bucket")
        G = len(caches)
        na = c0.n_pairs * G * c0.a * c0.rank
        self.data = torch.empty(na + c0.n_pairs * G * c0.b * c0.rank, dtype=torch.float32, device=c0.data.device)
        torch.cat([c.A for c in caches], dim=1, out=self.data[:na].view(c0.n_pairs, G * c0.a, c0.rank))
        torch.stack([c.B for c in caches], dim=1, out=self.data[na:].view(c0.n_pairs, G, c0.b, c0.rank))
        self.desc = _lib.FactorCacheDesc()
        self.desc.data = self.data.data_ptr()
        self.desc.key = c0.desc.key
        self.desc.true_epoch, self.desc.first_pair = c0.desc.true_epoch, c0.desc.first_pair
        self.desc.n_pairs, self.desc.rank = c0.n_pairs, c0.rank
        self.desc.a, self.desc.b = G * c0.a, G * c0.b
        self.n_groups, self.key = G, int(c0.desc.key)


def es_update(key: int, epoch: int, noise_reuse: int, rank: int, a: int, b: int, sigma: float,
              fitness_: torch.Tensor, first_thread: int = 0, n_total: Optional[int] = None,
              out: Optional[torch.Tensor] = None, cache: Optional[FactorCache] = None,
              mode: int = UPDATE_GRAD, sign_factors: bool = False, algo: int = ALGO_AUTO) -> torch.Tensor:
    """Fitness-weighted update of one LoRA-noised matrix.  mode UPDATE_RAW_ACC adds
    sum_i s_i A_i B_i^T (A_i scaled by sign*sigma/sqrt(rank)) to `out` instead."""
    _check(fitness_, "fitness", ndim=1)
    n = fitness_.numel()
    if out is None:
        if mode == UPDATE_RAW_ACC:
            out = torch.zeros((a, b), dtype=torch.float32, device=fitness_.device)
        else:
            out = torch.empty((a, b), dtype=torch.float32, device=fitness_.device)
    L = _lib.load()
    need = int(L.hses_es_update_workspace_bytes(a, b, rank, n))
    ws = _workspace(fitness_.device, need)
    ctx = get_context(fitness_.device)
    u = _lib.UpdateArgs()
    u.key, u.epoch, u.noise_reuse, u.first_thread = key & _U64, epoch, noise_reuse, first_thread
    u.n, u.n_total, u.rank, u.a, u.b, u.sigma = n, n if n_total is None else n_total, rank, a, b, sigma
    u.fitness, u.grad = fitness_.data_ptr(), out.data_ptr()
    u.workspace, u.workspace_bytes = (ws.data_ptr() if ws is not None else None), need
    if cache is not None:
        u.cache = C.pointer(cache.desc)
    u.mode = mode
    u.sign_factors = int(sign_factors)
    u.algo = algo
    _lib.check(L.hses_es_update_ex(ctx.handle, current_stream(), C.byref(u)))
    return out


def convert_fitnesses_bs(raw: torch.Tensor, group_size: int) -> torch.Tensor:
    """EggRollBS baseline-subtracted per-direction fitness (eggroll_bs.rs:226-250): (n,) -> (G,)."""
    _check(raw, "raw", ndim=1)
    n = raw.numel()
    if group_size < 1 or n % group_size:
        raise ValueError("n must be a positive multiple of group_size")
    out = torch.empty(group_size, dtype=torch.float32, device=raw.device)
    den = torch.empty(n // group_size, dtype=torch.float32, device=raw.device)
    ctx = get_context(raw.device)
    _lib.check(_lib.load().hses_convert_fitnesses_bs(ctx.handle, current_stream(), _ptr(raw), n, group_size,
                                                     _ptr(out), _ptr(den)))
    return out


def vector_mul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    _check(a, "a", ndim=1)
    _check(b, "b", ndim=1)
    if a.numel() != b.numel():
        raise ValueError("a and b must have the same length")
    out = torch.empty_like(a)
    ctx = get_context(a.device)
    _lib.check(_lib.load().hses_vector_mul(ctx.handle, current_stream(), _ptr(a), _ptr(b), _ptr(out), a.numel()))
    return out


def einsum_pair(a_t: torch.Tensor, b_t: torch.Tensor, scores: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """g_raw, g_ones of the paired einsum over explicit half-population factors:
    a_t (half, r, a), b_t (half, r, b) (innermost stride 1, outer strides free), scores (2*half,)."""
    _check(a_t, "a_t", ndim=3)
    _check(b_t, "b_t", ndim=3)
    _check(scores, "scores", ndim=1)
    half, r, a = a_t.shape
    if b_t.shape[:2] != (half, r):
        raise ValueError(f"b_t shape {tuple(b_t.shape)} does not match a_t {tuple(a_t.shape)}")
    b = b_t.shape[2]
    if half * r == 0:
        raise ValueError("einsum_pair: empty K")
    if scores.numel() != 2 * half:
        raise ValueError("scores must hold 2*half values")
    lib = _lib.load()
    ws = torch.empty(lib.hses_einsum_pair_workspace_bytes(half, r, a, b), dtype=torch.uint8, device=a_t.device)
    g_raw = torch.empty(a, b, dtype=torch.float32, device=a_t.device)
    g_ones = torch.empty_like(g_raw)
    ctx = get_context(a_t.device)
    _lib.check(lib.hses_einsum_pair(ctx.handle, current_stream(), _ptr(a_t), a_t.stride(0), a_t.stride(1), _ptr(b_t),
                                    b_t.stride(0), b_t.stride(1), _ptr(scores), half, r, a, b, _ptr(g_raw),
                                    _ptr(g_ones), _ptr(ws), ws.numel()))
    return g_raw, g_ones


def es_update_dense(key: int, epoch: int, noise_reuse: int, shape: Tuple[int, int], sigma: float,
                    fitness_: torch.Tensor, first_thread: int = 0,
                    n_total: Optional[int] = None) -> torch.Tensor:
    _check(fitness_, "fitness", ndim=1)
    n = fitness_.numel()
    out = torch.empty(shape, dtype=torch.float32, device=fitness_.device)
    ctx = get_context(fitness_.device)
    _lib.check(_lib.load().hses_es_update_dense(
        ctx.handle, current_stream(), C.c_uint64(key & _U64), epoch, noise_reuse, first_thread, n,
        n if n_total is None else n_total, shape[0] * shape[1], sigma, _ptr(fitness_), _ptr(out)))
    return out


def solver_step(kind: int, step: int, param: torch.Tensor, grad: torch.Tensor,
                m: Optional[torch.Tensor] = None, v: Optional[torch.Tensor] = None, lr: float = 0.01,
                beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
                weight_decay: float = 0.0, grad_scale: float = 1.0) -> None:
    """In-place optimizer step on a contiguous parameter tensor."""
    for t, name in ((param, "param"), (grad, "grad")):
        _check(t, name)
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    desc = _lib.SolverDesc(kind, lr, beta1, beta2, eps, weight_decay)
    ctx = get_context(param.device)
    _lib.check(_lib.load().hses_solver_step(ctx.handle, current_stream(), C.byref(desc), step,
                                            grad_scale, _ptr(param), _ptr(grad), _ptr(m), _ptr(v),
                                            param.numel()))


def base_sigma(sigma: float, rank: int) -> float:
    """sigma / sqrt(rank) in fp32, as the callers of get_lora_update_params compute it
    (eggroll.rs:365, 433)."""
    import numpy as np
    return float(np.float32(sigma) / np.sqrt(np.float32(rank)))


class HostPipeline:
    """Runs `perturbed_linear` for host-resident inputs and outputs.

    The population is cut into member chunks; the host-to-device copy of chunk c+1, the kernels
    of chunk c and the device-to-host copy of chunk c-1 run on three streams, so that a step
    costs about max(copy in, compute, copy out) instead of their sum.  `x_host` and `out_host`
    must be pinned.  Only single-time-step inputs (n_pop, bm, k) are cut this way.
    """

    def __init__(self, n_pop: int, bm: int, k: int, a: int, chunks: int = 8, device=None, taper: bool = False):
        ctx = get_context(device)
        self.dev = torch.device("cuda", ctx.device)
        if n_pop % (2 * chunks) != 0:
            raise ValueError("n_pop must be a multiple of 2*chunks (chunks hold whole antithetic pairs)")
        self.n_pop, self.bm, self.k, self.a = n_pop, bm, k, a
        self.sizes = self.chunk_sizes(n_pop, chunks, taper)
        self.chunks = len(self.sizes)
        self.mc = max(self.sizes)
        self.x_dev = [torch.empty((self.mc, bm, k), dtype=torch.float32, device=self.dev) for _ in range(2)]
        self.o_dev = [torch.empty((self.mc * bm, a), dtype=torch.float32, device=self.dev) for _ in range(2)]
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(self.dev) for _ in range(3))

    @staticmethod
    def chunk_sizes(n_pop: int, chunks: int, taper: bool):
        """Members per chunk (all even).  Tapered: the first chunk is an eighth of a regular one and
        the sizes double up to the regular size, mirrored at the end, so that the copy-in of the
        first chunk and the copy-out of the last one, which nothing overlaps, are short."""
        mc = n_pop // chunks
        if not taper:
            return [mc] * chunks
        head, s = [], max(2, (mc // 8) // 2 * 2)
        while s < mc:
            head.append(s)
            s *= 2
        rest = n_pop - 2 * sum(head)
        if rest <= 0:
            return [mc] * chunks
        mid = [mc] * (rest // mc) + ([rest % mc] if rest % mc else [])
        return head + mid + head[::-1]

    def run(self, x_host: torch.Tensor, param: torch.Tensor, out_host: torch.Tensor, first_thread: int = 0, **kw):
        if not (x_host.is_pinned() and out_host.is_pinned()):
            raise ValueError("x_host and out_host must be pinned host tensors")
        cur = torch.cuda.current_stream(self.dev)
        start = torch.cuda.Event()
        start.record(cur)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_event(start)
        ev_in, ev_run, ev_out = [], [], []
        lo = 0
        for c, m in enumerate(self.sizes):
            b = c & 1
            rows = m * self.bm
            with torch.cuda.stream(self.s_in):
                if c >= 2:
                    self.s_in.wait_event(ev_run[c - 2])      # the kernels of chunk c-2 have read x_dev[b]
                self.x_dev[b][:m].copy_(x_host[lo:lo + m], non_blocking=True)
                e = torch.cuda.Event(); e.record(self.s_in); ev_in.append(e)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(ev_in[c])
                if c >= 2:
                    self.s_run.wait_event(ev_out[c - 2])     # o_dev[b] has been copied out
                perturbed_linear(self.x_dev[b][:m], param, n_pop=m, bm=self.bm, first_thread=first_thread + lo,
                                 out=self.o_dev[b][:rows], **kw)
                e = torch.cuda.Event(); e.record(self.s_run); ev_run.append(e)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_run[c])
                out_host[lo * self.bm:lo * self.bm + rows].copy_(self.o_dev[b][:rows], non_blocking=True)
                e = torch.cuda.Event(); e.record(self.s_out); ev_out.append(e)
            lo += m
        cur.wait_event(ev_out[-1])
        cur.wait_event(ev_run[-1])
        return out_host


def wkv7(r, w, k, v, a, b, state: torch.Tensor, new_starts: Optional[torch.Tensor] = None) -> torch.Tensor:
    """rwkv7_inner_loop for a batch: inputs (n_seq, T, H, S); state (n_seq, H, S, S) is updated in place."""
    for t, name in ((r, "r"), (w, "w"), (k, "k"), (v, "v"), (a, "a"), (b, "b")):
        _check(t, name, ndim=4)
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    _check(state, "state", ndim=4)
    n_seq, T, H, S = r.shape
    if tuple(state.shape) != (n_seq, H, S, S) or not state.is_contiguous():
        raise ValueError("state must be a contiguous (n_seq, H, S, S) tensor")
    if new_starts is not None:
        _check(new_starts, "new_starts", torch.uint8, 2)
    out = torch.empty_like(r)
    ctx = get_context(r.device)
    _lib.check(_lib.load().hses_wkv7(ctx.handle, current_stream(), _ptr(r), _ptr(w), _ptr(k), _ptr(v), _ptr(a),
                                     _ptr(b), _ptr(new_starts), n_seq, T, H, S, _ptr(state), _ptr(out)))
    return out


def spiking_attention(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, heads: int, mode: int = 0,
                      beta: float = 1.0, tau_m: float = 2.0, v_th: float = 0.3, g_inh: float = 0.5,
                      n_iter: int = 8, want_weights: bool = False, beta_per_seq: Optional[torch.Tensor] = None):
    """Q, K, V: (n_seq, tokens, heads*head_dim) firing rates -> O of the same shape."""
    for t, name in ((Q, "Q"), (K, "K"), (V, "V")):
        _check(t, name, ndim=3)
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    n_seq, tokens, width = Q.shape
    if beta_per_seq is not None:
        _check(beta_per_seq, "beta_per_seq")
        if beta_per_seq.numel() != n_seq or not beta_per_seq.is_contiguous():
            raise ValueError("beta_per_seq must hold one contiguous value per sequence")
    if width % heads:
        raise ValueError("the model width must be a multiple of heads")
    O = torch.empty_like(Q)
    A = torch.empty((n_seq, heads, tokens, tokens), dtype=torch.float32, device=Q.device) if want_weights else None
    ctx = get_context(Q.device)
    _lib.check(_lib.load().hses_spiking_attention(ctx.handle, current_stream(), _ptr(Q), _ptr(K), _ptr(V), n_seq,
                                                  tokens, heads, width // heads, width, mode, beta, _ptr(beta_per_seq),
                                                  tau_m, v_th, g_inh, n_iter, _ptr(O), _ptr(A)))
    return (O, A) if want_weights else O


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """llm.rs:64-84: normalise the last axis (var = E[x^2] - E[x]^2), then weight and bias."""
    _check(x, "x")
    x = x.contiguous()
    c = x.shape[-1]
    out = torch.empty_like(x)
    ctx = get_context(x.device)
    _lib.check(_lib.load().hses_layer_norm(ctx.handle, current_stream(), _ptr(x), x.numel() // c, c,
                                           _ptr(weight.contiguous()), _ptr(bias.contiguous()), eps, _ptr(out)))
    return out


def group_norm(x: torch.Tensor, groups: int, weight: torch.Tensor, bias: torch.Tensor,
               eps: float = 1e-5) -> torch.Tensor:
    """GroupNorm.forward, llm.rs:90-145: x (n, c) or (n, c, l)."""
    _check(x, "x")
    if x.ndim not in (2, 3):
        raise ValueError("GroupNorm rank unsupported")
    x = x.contiguous()
    n, c = x.shape[0], x.shape[1]
    l = x.shape[2] if x.ndim == 3 else 1
    if c % groups:
        raise ValueError("channels must be a multiple of the group count")
    out = torch.empty_like(x)
    ctx = get_context(x.device)
    _lib.check(_lib.load().hses_group_norm(ctx.handle, current_stream(), _ptr(x), n, c, l, groups,
                                           _ptr(weight.contiguous()), _ptr(bias.contiguous()), eps, _ptr(out)))
    return out


def token_shift_mix(x: torch.Tensor, state: torch.Tensor, coef: torch.Tensor,
                    new_starts: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x + (prev - x) * coef with prev the previous row (row 0: state), 0 at new starts."""
    _check(x, "x", ndim=2)
    x = x.contiguous()
    T, c = x.shape
    out = torch.empty_like(x)
    ns = None
    if new_starts is not None:
        ns = new_starts.to(device=x.device, dtype=torch.uint8).contiguous()
    ctx = get_context(x.device)
    _lib.check(_lib.load().hses_token_shift_mix(ctx.handle, current_stream(), _ptr(x), T, c,
                                                _ptr(state.contiguous().view(-1)), _ptr(ns),
                                                _ptr(coef.contiguous().view(-1)), _ptr(out)))
    return out


def token_shift_mix_multi(x: torch.Tensor, state: torch.Tensor, coefs: Sequence[torch.Tensor],
                          new_starts: Optional[torch.Tensor] = None):
    """token_shift_mix for several coefficient vectors of one x (the six mixes of TimeMixing, llm.rs:381-392):
    x and its previous rows are read once.  Returns one tensor per coefficient vector."""
    _check(x, "x", ndim=2)
    x = x.contiguous()
    T, c = x.shape
    n = len(coefs)
    outs = [torch.empty_like(x) for _ in range(n)]
    cfs = [cf.contiguous().view(-1) for cf in coefs]
    ns = None
    if new_starts is not None:
        ns = new_starts.to(device=x.device, dtype=torch.uint8).contiguous()
    ctx = get_context(x.device)
    cp = (C.c_void_p * n)(*[t.data_ptr() for t in cfs])
    op = (C.c_void_p * n)(*[t.data_ptr() for t in outs])
    _lib.check(_lib.load().hses_token_shift_mix_multi(ctx.handle, current_stream(), _ptr(x), T, c,
                                                      _ptr(state.contiguous().view(-1)), _ptr(ns), n, cp, op))
    return outs


def rwkv_mix_prepare(w_lin, v_raw, v_lin, v_first, a_lin, k_raw, w0, v0, a0, k_k, k_a, H: int):
    """TimeMixing's element-wise work before the recurrence (llm.rs:396-440) in one pass: all (rows, C) dense.
    v_lin / v_first / v0 None: layer 0 (v = v_raw).  Returns (w, v, k, -kk, kk*a)."""
    rows, Cw = w_lin.shape
    S = Cw // H
    big = [w_lin, v_raw, a_lin, k_raw] + ([v_lin, v_first] if v_lin is not None else [])
    for t in big:
        _check(t, "input", ndim=2)
        if tuple(t.shape) != (rows, Cw) or not t.is_contiguous():
            raise ValueError("inputs must be contiguous (rows, H*S)")
    outs = [torch.empty_like(w_lin) for _ in range(5)]
    ctx = get_context(w_lin.device)
    c = lambda t: None if t is None else _ptr(t.contiguous())
    _lib.check(_lib.load().hses_rwkv_mix_prepare(ctx.handle, current_stream(), rows, H, S, _ptr(w_lin), _ptr(v_raw),
                                                 c(v_lin), c(v_first), _ptr(a_lin), _ptr(k_raw), c(w0), c(v0), c(a0),
                                                 c(k_k), c(k_a), *[_ptr(o) for o in outs]))
    return tuple(outs)


def rwkv_mix_finish(y_norm, r, k, v, gate, r_k, H: int) -> torch.Tensor:
    """(y_norm + (sum over each head of r * k * r_k) * v) * gate, llm.rs:462-472; (rows, C) dense."""
    rows, Cw = y_norm.shape
    for t in (y_norm, r, k, v, gate):
        _check(t, "input", ndim=2)
        if tuple(t.shape) != (rows, Cw) or not t.is_contiguous():
            raise ValueError("inputs must be contiguous (rows, H*S)")
    out = torch.empty_like(y_norm)
    ctx = get_context(y_norm.device)
    _lib.check(_lib.load().hses_rwkv_mix_finish(ctx.handle, current_stream(), rows, H, Cw // H, _ptr(y_norm), _ptr(r),
                                                _ptr(k), _ptr(v), _ptr(gate), _ptr(r_k.contiguous()), _ptr(out)))
    return out


def relu_square(x: torch.Tensor) -> torch.Tensor:
    _check(x, "x")
    x = x.contiguous()
    out = torch.empty_like(x)
    ctx = get_context(x.device)
    _lib.check(_lib.load().hses_relu_square(ctx.handle, current_stream(), _ptr(x), x.numel(), _ptr(out)))
    return out


def rate_encode(p: torch.Tensor, gain: float) -> torch.Tensor:
    """snn_transformer.rs:109-116: sigmoid(gain * p / (1 + |p|))."""
    _check(p, "p")
    p = p.contiguous()
    out = torch.empty_like(p)
    ctx = get_context(p.device)
    _lib.check(_lib.load().hses_rate_encode(ctx.handle, current_stream(), _ptr(p), p.numel(), gain, _ptr(out)))
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, pos: Optional[torch.Tensor] = None,
              A: Optional[torch.Tensor] = None, B: Optional[torch.Tensor] = None,
              rows_per_member: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """do_emb over a population: ids (rows,) int32 -> (rows, d) = table[ids] + A_m[ids] B_m^T + pos[row % L].
    A (n, vocab, r) scaled by sign*sigma/sqrt(r) and B (n, d, r) as lora_factors returns them for a
    parameter of shape (vocab, d); member m owns rows_per_member consecutive rows."""
    _check(table, "table", ndim=2)
    if ids.dtype != torch.int32 or not ids.is_cuda or not ids.is_contiguous():
        raise ValueError("ids must be a contiguous CUDA int32 tensor")
    rows = ids.numel()
    vocab, d = table.shape
    rank = 0
    if A is not None:
        _check(A, "A", ndim=3)
        _check(B, "B", ndim=3)
        if A.shape[1] != vocab or B.shape[1] != d or A.shape[2] != B.shape[2] or A.shape[0] != B.shape[0]:
            raise ValueError("A must be (n, vocab, r) and B (n, d, r)")
        if not (A.is_contiguous() and B.is_contiguous()):
            raise ValueError("A and B must be contiguous")
        rank = A.shape[2]
        if rows_per_member < 1 or rows != A.shape[0] * rows_per_member:
            raise ValueError("rows must equal members * rows_per_member")
    L = 0
    if pos is not None:
        _check(pos, "pos", ndim=2)
        if pos.shape[1] != d or not pos.is_contiguous():
            raise ValueError("pos must be a contiguous (L, d) tensor")
        L = pos.shape[0]
    if out is None:
        out = torch.empty((rows, d), dtype=torch.float32, device=table.device)
    ctx = get_context(table.device)
    _lib.check(_lib.load().hses_embedding(ctx.handle, current_stream(), ids.data_ptr(), rows, _ptr(table), table.stride(0),
                                          vocab, d, _ptr(pos), L, _ptr(A), _ptr(B), rank, rows_per_member, _ptr(out),
                                          out.stride(0)))
    return out


def lif_rate(cur: torch.Tensor, T: int, tau_m: float, v_th: float, reset_mode: int = RESET_HARD,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Firing rate over T steps of LIF neurons driven by the constant currents `cur` (any shape, dense)."""
    _check(cur, "cur")
    if not cur.is_contiguous():
        raise ValueError("cur must be contiguous")
    if out is None:
        out = torch.empty_like(cur)
    ctx = get_context(cur.device)
    _lib.check(_lib.load().hses_lif_rate(ctx.handle, current_stream(), _ptr(cur), cur.numel(), T, tau_m, v_th, reset_mode,
                                         _ptr(out)))
    return out


def swish(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _check(x, "x")
    if not x.is_contiguous():
        raise ValueError("x must be contiguous")
    if out is None:
        out = torch.empty_like(x)
    ctx = get_context(x.device)
    _lib.check(_lib.load().hses_swish(ctx.handle, current_stream(), _ptr(x), x.numel(), _ptr(out)))
    return out


def add_inplace(acc: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    _check(acc, "acc")
    _check(y, "y")
    if acc.shape != y.shape or not (acc.is_contiguous() and y.is_contiguous()):
        raise ValueError("acc and y must be contiguous tensors of one shape")
    ctx = get_context(acc.device)
    _lib.check(_lib.load().hses_add_inplace(ctx.handle, current_stream(), _ptr(acc), _ptr(y), acc.numel()))
    return acc


def token_fitness(logits: torch.Tensor, ids: torch.Tensor, n_members: int, seqs: int, L: int,
                  gain: float = 1.0) -> torch.Tensor:
    """Per member the mean next-token log-likelihood: logits (n_members*seqs*L, vocab), ids the
    int32 tokens in the same row order; position t is scored against the token at t+1."""
    _check(logits, "logits", ndim=2)
    rows, vocab = logits.shape
    if rows != n_members * seqs * L or ids.numel() != rows or ids.dtype != torch.int32:
        raise ValueError("logits and ids must hold n_members*seqs*L rows")
    scratch = torch.empty(rows, dtype=torch.float32, device=logits.device)
    out = torch.empty(n_members, dtype=torch.float32, device=logits.device)
    ctx = get_context(logits.device)
    _lib.check(_lib.load().hses_token_fitness(ctx.handle, current_stream(), _ptr(logits), logits.stride(0), ids.data_ptr(),
                                              n_members, seqs, L, vocab, gain, _ptr(scratch), _ptr(out)))
    return out
