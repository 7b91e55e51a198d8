"""Host-side mirror of hyperscalees-models/src/snn.rs for the SNN MLP path.

`lif_step`, `run_lif` and `SnnModel` keep the reference's names and argument
order; `SnnMlp` generalises the fixed two-hidden-layer model to a list of
layer widths (the reference's Python trainers use variable depth).  Forward
passes run whole populations per launch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import ops
from .noiser import MM_PARAM, PARAM, FrozenNoiserParams, NoiserParams


@dataclass(frozen=True)
class LifParams:
    """snn.rs:31-36."""
    tau_m: float
    v_th: float


def lif_step(tau_m: float, v_th: float, v: torch.Tensor, current: torch.Tensor,
             reset_mode: int = ops.RESET_HARD):
    """snn.rs:53-65: returns (new_v, spike); inputs are left untouched."""
    shape = current.shape
    cur = current.reshape(1, -1, shape[-1]) if current.dim() >= 2 else current.reshape(1, 1, -1)
    new_v = v.detach().clone().reshape(cur.shape[1], cur.shape[2]).contiguous()
    spikes = ops.lif_scan(cur.contiguous(), tau_m, v_th, v=new_v, reset_mode=reset_mode)
    return new_v.reshape(shape), spikes.reshape(shape)


def run_lif(params: LifParams, input_current: torch.Tensor, v0: Optional[torch.Tensor],
            reset_mode: int = ops.RESET_HARD) -> torch.Tensor:
    """snn.rs:73-97: input_current (T, batch, hidden) -> spikes (T, batch, hidden)."""
    v = None if v0 is None else v0.detach().clone()
    return ops.lif_scan(input_current, params.tau_m, params.v_th, v=v, reset_mode=reset_mode)


def default_base_keys(n: int) -> List[int]:
    """(i+1) * 0x9E3779B97F4A7C15 mod 2^64, hyperscalees/src/snn_mnist_train.rs:126-128."""
    return [((i + 1) * 0x9E3779B97F4A7C15) & ((1 << 64) - 1) for i in range(n)]


class SnnMlp:
    """SNN classifier: perturbed linear -> LIF per hidden layer, rate readout, gain.

    Parameters are kept in the reference's order `[fc..., out_gain]`
    (snn.rs:235-245) with es classes `[MM_PARAM..., PARAM]`.
    """

    def __init__(self, dims: Sequence[int], device=None, tau_m: float = 20.0, v_th: float = 0.3,
                 reset_mode: int = ops.RESET_HARD, seed: int = 0):
        from .core import default_device
        self.device = torch.device(device) if device is not None else default_device()
        self.dims = list(dims)
        g = np.random.Generator(np.random.PCG64(seed))
        # Mm::new: N(0, 1/sqrt(in)) (hyperscalees-models/src/common.rs:113-121)
        self.weights: List[torch.Tensor] = []
        for i in range(len(dims) - 1):
            w = g.standard_normal((dims[i + 1], dims[i])).astype(np.float32) / np.float32(np.sqrt(dims[i]))
            self.weights.append(torch.as_tensor(w, device=self.device))
        self.out_gain = torch.ones((1, 1), dtype=torch.float32, device=self.device)
        self.tau_m, self.v_th, self.reset_mode = tau_m, v_th, reset_mode

    def params(self) -> List[torch.Tensor]:
        return list(self.weights) + [self.out_gain]

    def es_map(self) -> List[int]:
        return [MM_PARAM] * len(self.weights) + [PARAM]

    def set_params(self, params: Sequence[torch.Tensor]) -> None:
        self.weights = [p for p in params[:len(self.weights)]]
        self.out_gain = params[len(self.weights)]

    def forward_population(self, x: torch.Tensor, frozen: Optional[FrozenNoiserParams] = None,
                           noiser: Optional[NoiserParams] = None,
                           base_keys: Optional[Sequence[int]] = None, epoch: int = 0,
                           first_thread: int = 0, want_hidden: bool = False, algo: int = ops.ALGO_AUTO):
        """x: (T, n_pop, bm, in) spikes.  Returns logits (n_pop*bm, classes); member i is
        perturbed with thread id first_thread + i (clean forward when frozen is None)."""
        T, n_pop, bm, _ = x.shape
        perturb = frozen is not None
        kw = dict(n_pop=n_pop, bm=bm, perturb=perturb, algo=algo)
        if perturb:
            kw.update(sigma=noiser.sigma, rank=frozen.rank, epoch=epoch, first_thread=first_thread,
                      noise_reuse=frozen.noise_reuse)
        cur_in = x
        n_rows = n_pop * bm
        hidden = None
        for l, w in enumerate(self.weights[:-1]):
            key = base_keys[l] if perturb else 0
            cur = ops.perturbed_linear(cur_in, w, t_steps=T, key=key, **kw)
            spikes = ops.lif_scan(cur.view(T, n_rows, w.shape[0]), self.tau_m, self.v_th,
                                  reset_mode=self.reset_mode)
            cur_in = spikes
            hidden = spikes
        rate = ops.time_mean(cur_in.reshape(T, n_rows, cur_in.shape[-1]))
        key = base_keys[len(self.weights) - 1] if perturb else 0
        gain = float(self.out_gain.reshape(-1)[0].item())
        logits = ops.perturbed_linear(rate, self.weights[-1], t_steps=1, key=key, out_scale=gain, **kw)
        return (logits, hidden) if want_hidden else logits


class SnnModel(SnnMlp):
    """The reference's fixed two-hidden-layer model (snn.rs:188-282)."""

    def __init__(self, in_dim: int, hidden1: int, hidden2: int, num_classes: int, device=None,
                 seed: int = 0):
        super().__init__([in_dim, hidden1, hidden2, num_classes], device=device, seed=seed)

    def forward(self, x: torch.Tensor, noise=None) -> torch.Tensor:
        """snn.rs:253-282: x (T, batch, in_dim) -> logits (batch, classes).  `noise` is
        either None (clean) or a tuple (frozen, noiser, base_keys, IterInfo): the whole
        batch is then evaluated as ONE member, like the reference's closure path."""
        T, batch, in_dim = x.shape
        xx = x.reshape(T, 1, batch, in_dim)
        if noise is None:
            return self.forward_population(xx)
        frozen, noiser, base_keys, info = noise
        return self.forward_population(xx, frozen, noiser, base_keys, epoch=info.epoch,
                                       first_thread=info.thread_id)


class PopulationStep:
    """Drives the composite C entry points (`hses_population_eval` / `hses_population_update`):
    encode -> perturbed forward -> fitness on this rank's shard, then — after the caller has
    all-gathered the raw fitness when several GPUs share the population — z-score, noise-
    regenerating update of every layer and the solver step, all enqueued on the current stream
    without host round-trips.  Parameters (and Adam moments) live on the device and are updated
    in place; `out_gain` is read from its device tensor by the readout."""

    def __init__(self, net: SnnMlp, frozen: FrozenNoiserParams, noiser: NoiserParams,
                 base_keys: Sequence[int], T: int, n_pop: int, bm: int, first_thread: int = 0,
                 reward: int = ops.REWARD_LOGLIK, cache: str = "off", n_total: Optional[int] = None):
        import ctypes as C
        from . import _lib
        from .core import get_context
        self.C, self._lib, self.L = C, _lib, _lib.load()
        self.net, self.frozen, self.noiser = net, frozen, noiser
        self.keys = [int(k) & ((1 << 64) - 1) for k in base_keys]
        self.T, self.n_pop, self.bm, self.first_thread, self.reward = T, n_pop, bm, first_thread, reward
        self.ctx = get_context(net.device)
        self.params = [w.contiguous() for w in net.weights] + [net.out_gain.contiguous()]
        net.weights, net.out_gain = self.params[:-1], self.params[-1]
        kind = frozen.solver.kind
        self.moments = None
        if kind in ("adam", "adamw"):
            self.moments = ([torch.zeros_like(p) for p in self.params], [torch.zeros_like(p) for p in self.params])
        self._ws = None
        self.caches = None
        # "auto": generate every layer's factors once per epoch bucket (at the first eval of the
        # bucket) and let the forward pass and the update read them; with noise_reuse == 0 the
        # bucket never changes, so the generation cost is paid once per run
        if cache not in ("off", "auto"):
            raise ValueError("cache must be 'off' or 'auto'")
        self.cache_policy, self.n_total, self._cache_bucket = cache, n_total, None

    def build_caches(self, epoch: int = 0, n_total: Optional[int] = None) -> int:
        """Generates the factors of every layer once and keeps them on the device
        (LoraNoiseCache, eggroll.rs:229-309); eval() and update() then read them instead of
        regenerating.  Covers the whole population when n_total is given (needed for update()),
        else this shard's members.  Valid until the epoch bucket changes; returns the bytes held."""
        if n_total is None:
            first_pair = self.first_thread // 2
            n_pairs = (self.first_thread + self.n_pop - 1) // 2 - first_pair + 1
        else:
            first_pair, n_pairs = 0, n_total // 2
        self.caches = [ops.FactorCache(self.keys[l], epoch, self.frozen.noise_reuse, self.frozen.rank,
                                       w.shape[0], w.shape[1], n_pairs, first_pair, device=self.net.device)
                       for l, w in enumerate(self.net.weights)]
        return sum(c.data.numel() * 4 for c in self.caches)

    def drop_caches(self) -> None:
        self.caches = None

    def _model(self):
        C, _lib = self.C, self._lib
        n = len(self.net.weights)
        dims = (C.c_int32 * (n + 1))(*self.net.dims)
        wp = (C.c_void_p * n)(*[w.data_ptr() for w in self.net.weights])
        ws = (C.c_int64 * n)(*[w.stride(0) for w in self.net.weights])
        keys = (C.c_uint64 * n)(*self.keys[:n])
        vth = (C.c_float * max(n - 1, 1))(*([self.net.v_th] * max(n - 1, 1)))
        cp = None
        if self.caches is not None:
            cp = (C.POINTER(_lib.FactorCacheDesc) * n)(*[C.pointer(c.desc) for c in self.caches])
        m = _lib.SnnModelDesc(n, dims, wp, ws, keys, 1.0, self.net.out_gain.data_ptr(), self.net.tau_m, vth,
                              self.net.reset_mode, cp)
        self._keep = (dims, wp, ws, keys, vth, cp)
        return m

    def _args(self, epoch: int, perturb: bool = True):
        return self._lib.PopArgs(self.T, self.n_pop, self.bm, int(perturb), self.noiser.sigma, self.frozen.rank,
                                 epoch, self.first_thread, self.frozen.noise_reuse)

    def _scratch(self, nbytes: int) -> torch.Tensor:
        if self._ws is None or self._ws.numel() < nbytes + 256:
            self._ws = torch.empty(nbytes + 256, dtype=torch.uint8, device=self.net.device)
        off = (-self._ws.data_ptr()) % 256
        return self._ws[off:off + nbytes]

    def eval(self, images: torch.Tensor, labels: torch.Tensor, seeds: Sequence[int], epoch: int = 0,
             want_logits: bool = False, perturb: bool = True):
        """images (n_pop*bm, in) probabilities, labels int32 -> raw fitness (n_pop,)."""
        C = self.C
        if self.cache_policy == "auto" and perturb:
            nr = self.frozen.noise_reuse
            bucket = 0 if nr == 0 else epoch // nr
            if bucket != self._cache_bucket:
                self.caches = None   # release the old bucket before allocating the new one
                self.build_caches(epoch, self.n_total)
                self._cache_bucket = bucket
        m, p = self._model(), self._args(epoch, perturb)
        need = int(self.L.hses_population_eval_workspace_bytes(C.byref(m), C.byref(p)))
        ws = self._scratch(need)
        raw = torch.empty(self.n_pop, dtype=torch.float32, device=images.device)
        logits = torch.empty((self.n_pop * self.bm, self.net.dims[-1]), dtype=torch.float32,
                             device=images.device) if want_logits else None
        sd = (C.c_uint32 * 4)(*[int(s) & 0xFFFFFFFF for s in seeds])
        from .core import current_stream
        self._lib.check(self.L.hses_population_eval(
            self.ctx.handle, current_stream(), C.byref(m), C.byref(p), images.data_ptr(),
            images.stride(0), labels.data_ptr(), sd, self.reward, raw.data_ptr(),
            logits.data_ptr() if want_logits else None, ws.data_ptr(), need))
        return (raw, logits) if want_logits else raw

    def update_sharded(self, raw_fitness: torch.Tensor, epoch: int = 0, gain_key: Optional[int] = None,
                       group=None, reduce_fn=None, comm=None) -> None:
        """Like update(), but this rank only contracts the factors of ITS members (first_thread ..
        first_thread + n_pop - 1); the partial gradients of all parameters are summed with one
        all-reduce (through `comm`, the library's own communicator, when given; else through
        torch.distributed when it is initialised) and every rank applies the same solver
        step, so parameters stay identical on all ranks.  reduce_fn(grads), when given, replaces
        the all-reduce (it must leave the sum over all shards in `grads`)."""
        import torch.distributed as dist
        C = self.C
        m = self._model()
        n_total = raw_fitness.numel()
        need = int(self.L.hses_population_update_workspace_bytes(C.byref(m), self.frozen.rank, n_total))
        ws = self._scratch(need)
        elems = int(self.L.hses_population_grads_elems(C.byref(m)))
        if getattr(self, "_grads", None) is None or self._grads.numel() != elems:
            self._grads = torch.empty(elems, dtype=torch.float32, device=self.net.device)
        gk = self.keys[len(self.net.weights)] if gain_key is None else gain_key
        from .core import current_stream
        self._lib.check(self.L.hses_population_grads(
            self.ctx.handle, current_stream(), C.byref(m), self.noiser.sigma, self.frozen.rank, epoch,
            self.frozen.noise_reuse, self.frozen.group_size, int(self.frozen.freeze_nonlora),
            C.c_uint64(gk & ((1 << 64) - 1)), raw_fitness.data_ptr(), n_total, self.first_thread, self.n_pop,
            self._grads.data_ptr(), ws.data_ptr(), need))
        if reduce_fn is not None:
            reduce_fn(self._grads)
        elif comm is not None:
            if comm.world > 1:
                comm.allreduce_grads(self._grads)
        elif dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(self._grads, op=dist.ReduceOp.SUM, group=group)
        sv = self.frozen.solver
        kind = {"sgd": ops.SGD, "adam": ops.ADAM, "adamw": ops.ADAMW}[sv.kind]
        desc = self._lib.SolverDesc(kind, sv.lr, sv.beta1, sv.beta2, sv.eps, sv.weight_decay if kind == ops.ADAMW else 0.0)
        if kind != ops.SGD:
            self.noiser.opt_state.step += 1
        n = len(self.params)
        pp = (C.c_void_p * n)(*[t.data_ptr() for t in self.params])
        mp = vp = None
        if self.moments is not None:
            mp = (C.c_void_p * n)(*[t.data_ptr() for t in self.moments[0]])
            vp = (C.c_void_p * n)(*[t.data_ptr() for t in self.moments[1]])
        self._lib.check(self.L.hses_population_apply(
            self.ctx.handle, current_stream(), C.byref(m), C.byref(desc), self.noiser.opt_state.step, pp, mp, vp,
            self._grads.data_ptr()))

    def update(self, raw_fitness: torch.Tensor, epoch: int = 0, gain_key: Optional[int] = None) -> None:
        """raw_fitness: the FULL population's raw fitness (thread ids 0..n-1). Updates parameters in place."""
        C = self.C
        m = self._model()
        n_total = raw_fitness.numel()
        need = int(self.L.hses_population_update_workspace_bytes(C.byref(m), self.frozen.rank, n_total))
        ws = self._scratch(need)
        sv = self.frozen.solver
        kind = {"sgd": ops.SGD, "adam": ops.ADAM, "adamw": ops.ADAMW}[sv.kind]
        desc = self._lib.SolverDesc(kind, sv.lr, sv.beta1, sv.beta2, sv.eps, sv.weight_decay if kind == ops.ADAMW else 0.0)
        if kind != ops.SGD:
            self.noiser.opt_state.step += 1
        n = len(self.params)
        pp = (C.c_void_p * n)(*[t.data_ptr() for t in self.params])
        mp = vp = None
        if self.moments is not None:
            mp = (C.c_void_p * n)(*[t.data_ptr() for t in self.moments[0]])
            vp = (C.c_void_p * n)(*[t.data_ptr() for t in self.moments[1]])
        gk = self.keys[len(self.net.weights)] if gain_key is None else gain_key
        from .core import current_stream
        self._lib.check(self.L.hses_population_update(
            self.ctx.handle, current_stream(), C.byref(m), self.noiser.sigma, self.frozen.rank, epoch,
            self.frozen.noise_reuse, self.frozen.group_size, int(self.frozen.freeze_nonlora),
            C.c_uint64(gk & ((1 << 64) - 1)), raw_fitness.data_ptr(), n_total, C.byref(desc),
            self.noiser.opt_state.step, pp, mp, vp, ws.data_ptr(), need))


class ChannelMixing:
    """RWKV-7 ChannelMixing (hyperscalees-models/src/llm.rs:177-213): token shift with the
    per-channel strength x_k, key projection, relu^2, value projection; bias-free Linear layers
    (x @ W^T).  With `noise` = (noiser, frozen, params, base keys, iterinfo) the two projections
    go through the noiser's do_mm, i.e. they carry the member's rank-r perturbation like every
    MM weight of the reference's JAX model."""

    def __init__(self, x_k: torch.Tensor, key_weight: torch.Tensor, value_weight: torch.Tensor):
        self.x_k, self.key_weight, self.value_weight = x_k, key_weight, value_weight

    def forward(self, x: torch.Tensor, state: torch.Tensor, length: int,
                new_starts: Optional[torch.Tensor] = None, noise=None):
        xk = ops.token_shift_mix(x, state, self.x_k, new_starts)
        if noise is None:
            k = ops.perturbed_linear(xk, self.key_weight, n_pop=1, bm=xk.shape[0], perturb=False)
            k = ops.relu_square(k)
            out = ops.perturbed_linear(k, self.value_weight, n_pop=1, bm=k.shape[0], perturb=False)
        else:
            nz, frozen, params, keys, info = noise
            k = ops.relu_square(nz.do_mm(frozen, params, self.key_weight, keys[0], info, xk))
            out = nz.do_mm(frozen, params, self.value_weight, keys[1], info, k)
        return out, x[length - 1:length].clone()


class TimeMixing:
    """RWKV-7 TimeMixing (hyperscalees-models/src/llm.rs:298-479) for one sequence x (T, C).

    `weights` holds the reference's fields by name: vectors x_r, x_w, x_k, x_v, x_a, x_g, w0, v0,
    a0, k_k, k_a (C,), r_k (H, S) or (C,); Linear weights receptance, key, value, output (C, C) as
    (out, in); Tmm weights w1, v1, a1, g1 (C, k) and w2, v2, a2, g2 (k, C) as (in, out); ln_x_weight
    and ln_x_bias (C,).  Token shifts, every projection, the recurrence and the per-head group norm
    run through the library's kernels; gates and the readout bonus are tensor arithmetic.  With
    `noise` = (noiser, frozen, params, {name: base key}, iterinfo) the Linear and Tmm products go
    through the noiser's do_mm / do_Tmm and carry the member's rank-r perturbation."""

    def __init__(self, weights: dict):
        self.w = dict(weights)
        # x @ W for the Tmm weights runs as x @ (W^T)^T through the clean linear kernel
        self._t = {n: self.w[n].t().contiguous() for n in ("w1", "w2", "v1", "v2", "a1", "a2", "g1", "g2")
                   if n in self.w}

    def _linear(self, name: str, x: torch.Tensor, noise) -> torch.Tensor:
        if noise is None:
            return ops.perturbed_linear(x.contiguous(), self.w[name], n_pop=1, bm=x.shape[0], perturb=False)
        nz, frozen, params, keys, info = noise
        return nz.do_mm(frozen, params, self.w[name], keys[name], info, x.contiguous())

    def _tmm(self, name: str, x: torch.Tensor, noise) -> torch.Tensor:
        if noise is None:
            return ops.perturbed_linear(x.contiguous(), self._t[name], n_pop=1, bm=x.shape[0], perturb=False)
        nz, frozen, params, keys, info = noise
        return nz.do_Tmm(frozen, params, self.w[name], keys[name], info, x.contiguous())

    def forward(self, x: torch.Tensor, state: torch.Tensor, v_first: torch.Tensor, length: int,
                new_starts: Optional[torch.Tensor], h: int, s_dim: int, layer_id: int, noise=None):
        """x (T, C); state (1 + S, C): row 0 the previous token, rows 1.. the (H, S, S) recurrent
        state flattened; returns (out (T, C), new state, v_first)."""
        w = self.w
        T, C = x.shape
        x = x.contiguous()
        prev = state[0].contiguous()
        ns = None if new_starts is None else new_starts.to(device=x.device, dtype=torch.uint8).contiguous()
        mix = lambda name: ops.token_shift_mix(x, prev, w[name], ns)
        xr, xw, xk, xv, xa, xg = (mix(n) for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g"))

        r = self._linear("receptance", xr, noise)
        inner_w = w["w0"].unsqueeze(0) + self._tmm("w2", torch.tanh(self._tmm("w1", xw, noise)), noise)
        wdec = -torch.nn.functional.softplus(-inner_w) - 0.5
        k = self._linear("key", xk, noise)
        v = self._linear("value", xv, noise)
        if layer_id == 0:
            v_first = v.clone()
        else:
            sig = torch.sigmoid(w["v0"].unsqueeze(0) + self._tmm("v2", torch.tanh(self._tmm("v1", xv, noise)), noise))
            v = v + (v_first - v) * sig
        a = torch.sigmoid(w["a0"].unsqueeze(0) + self._tmm("a2", torch.tanh(self._tmm("a1", xa, noise)), noise))
        g = self._tmm("g2", torch.sigmoid(self._tmm("g1", xg, noise)), noise)

        kk3 = (k * w["k_k"].unsqueeze(0)).view(T, h, s_dim)
        kk = (kk3 / kk3.pow(2).sum(dim=2, keepdim=True).sqrt().clamp_min(1e-12)).reshape(T, C)
        k = k * (w["k_a"].unsqueeze(0) * (a - 1.0) + 1.0)

        new_state = state.clone()
        new_state[0] = x[length - 1]
        s_run = state[1:1 + s_dim].reshape(1, h, s_dim, s_dim).contiguous().clone()
        shp = lambda t_: t_.reshape(1, T, h, s_dim).contiguous()
        r4, w4, k4, v4, a4, b4 = shp(r), shp(wdec), shp(k), shp(v), shp(-kk), shp(kk * a)
        nsb = None if ns is None else ns.view(1, T)
        if length >= T:
            out = ops.wkv7(r4, w4, k4, v4, a4, b4, s_run, nsb)
            s_keep = s_run
        else:
            # the state handed back is the one after token length-1; later tokens still produce outputs
            cut = lambda t_, lo, hi: t_[:, lo:hi].contiguous()
            o1 = ops.wkv7(*(cut(t_, 0, length) for t_ in (r4, w4, k4, v4, a4, b4)), s_run,
                          None if nsb is None else nsb[:, :length].contiguous())
            s_keep = s_run.clone()
            o2 = ops.wkv7(*(cut(t_, length, T) for t_ in (r4, w4, k4, v4, a4, b4)), s_run,
                          None if nsb is None else nsb[:, length:].contiguous())
            out = torch.cat([o1, o2], dim=1)
        new_state[1:1 + s_dim] = s_keep.reshape(s_dim, C)

        y = ops.group_norm(out.reshape(T, C), h, w["ln_x_weight"], w["ln_x_bias"], eps=64e-5)
        bonus = (r.view(T, h, s_dim) * k.view(T, h, s_dim) * w["r_k"].reshape(1, h, s_dim)).sum(dim=2, keepdim=True)
        y = y + (bonus * v.view(T, h, s_dim)).reshape(T, C)
        y = y * g
        return self._linear("output", y, noise), new_state, v_first
