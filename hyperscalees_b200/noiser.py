"""Host-side mirror of the hyperscalees-noiser crate for the EggRoll path.

Names, argument meaning and error behaviour follow
hyperscalees-noiser/src/noiser.rs and eggroll.rs; tensors are torch CUDA
tensors and every computation is a call into the CUDA library.  The Rust
crate's per-member entry points are kept, and population-wide forms (one
launch for all members) are added beside them because that is how the
device path is meant to be driven.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import ops

# es-class constants, hyperscalees-models/src/common.rs:15-21
PARAM, MM_PARAM, EMB_PARAM, EXCLUDED = 0, 1, 2, 3


@dataclass(frozen=True)
class IterInfo:
    """noiser.rs:24-28."""
    epoch: int
    thread_id: int


# ---------------------------------------------------------------------------
# Solver (noiser.rs:42-244)
# ---------------------------------------------------------------------------
@dataclass
class MomentState:
    m: torch.Tensor
    v: torch.Tensor


@dataclass
class OptimizerState:
    step: int = 0
    moments: List[MomentState] = field(default_factory=list)


@dataclass
class Solver:
    kind: str  # "sgd" | "adam" | "adamw" | "trust_region"
    lr: float = 0.0
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0
    max_norm: float = 0.0
    inner: Optional["Solver"] = None

    @staticmethod
    def sgd(lr: float) -> "Solver":
        return Solver("sgd", lr=lr)

    @staticmethod
    def adam(lr: float) -> "Solver":
        return Solver("adam", lr=lr)

    @staticmethod
    def adamw(lr: float) -> "Solver":
        return Solver("adamw", lr=lr, weight_decay=1e-4)

    @staticmethod
    def trust_region(max_norm: float, inner: "Solver") -> "Solver":
        return Solver("trust_region", max_norm=max_norm, inner=inner)

    def init_state(self, params: Sequence[torch.Tensor]) -> OptimizerState:
        if self.kind == "sgd":
            return OptimizerState(0, [])
        if self.kind == "trust_region":
            return self.inner.init_state(params)
        return OptimizerState(0, [MomentState(torch.zeros_like(p), torch.zeros_like(p)) for p in params])

    def update(self, params: Sequence[torch.Tensor], grads: Sequence[torch.Tensor],
               state: OptimizerState, grad_scale: float = 1.0) -> List[torch.Tensor]:
        """Returns updated copies; the inputs are left untouched (noiser.rs:155-159)."""
        if self.kind == "trust_region":
            # clip_by_global_norm (noiser.rs:232-244): one scale for all gradients
            sq = sum(float((g.double() ** 2).sum()) for g in grads)
            norm = float(np.sqrt(np.float32(sq)))
            scale = self.max_norm / norm if (norm > self.max_norm and norm > 0.0) else 1.0
            return self.inner.update(params, grads, state, grad_scale=scale)
        kind = {"sgd": ops.SGD, "adam": ops.ADAM, "adamw": ops.ADAMW}[self.kind]
        if kind != ops.SGD:
            state.step += 1
        out = []
        for i, (p, g) in enumerate(zip(params, grads)):
            q = p.detach().clone().contiguous()
            m = v = None
            if kind != ops.SGD:
                m, v = state.moments[i].m, state.moments[i].v
            ops.solver_step(kind, state.step, q, g.contiguous(), m, v, lr=self.lr, beta1=self.beta1,
                            beta2=self.beta2, eps=self.eps,
                            weight_decay=self.weight_decay if kind == ops.ADAMW else 0.0,
                            grad_scale=grad_scale)
            out.append(q)
        return out


@dataclass
class FrozenNoiserParams:
    """noiser.rs:248-260."""
    group_size: int
    freeze_nonlora: bool
    noise_reuse: int
    rank: int
    solver: Solver


@dataclass
class NoiserParams:
    """noiser.rs:263-269."""
    sigma: float
    opt_state: OptimizerState


def init_noiser(params: Sequence[torch.Tensor], sigma: float, _lr: float, group_size: int,
                freeze_nonlora: bool, noise_reuse: int, rank: int,
                solver: Solver) -> Tuple[FrozenNoiserParams, NoiserParams]:
    """eggroll.rs:28-51."""
    frozen = FrozenNoiserParams(group_size, freeze_nonlora, noise_reuse, rank, solver)
    return frozen, NoiserParams(sigma, solver.init_state(params))


# ---------------------------------------------------------------------------
# RNG helpers
# ---------------------------------------------------------------------------
def noise_seed(key: int, true_epoch: int, true_thread: int) -> int:
    """noiser.rs:495-506."""
    return ops.noise_seed(key, true_epoch, true_thread)


def epoch_thread_sign(info: IterInfo, noise_reuse: int) -> Tuple[int, int, float]:
    """eggroll.rs:60-65 (integer division truncates toward zero, as in Rust)."""
    true_epoch = 0 if noise_reuse == 0 else int(info.epoch / noise_reuse)
    true_thread = int(info.thread_id / 2)
    sign = 1.0 if info.thread_id % 2 == 0 else -1.0
    return true_epoch, true_thread, sign


class DeterministicNoise:
    """noiser.rs:436-490.  `normal_tensor` continues the stream across calls, as the
    Rust struct does, by remembering how many normals were consumed."""

    def __init__(self, seed: int):
        self.seed = seed
        self._consumed = 0

    def normal_tensor(self, shape: Sequence[int], device=None) -> torch.Tensor:
        n = int(np.prod(shape))
        flat = ops.normal_fill(self.seed, self._consumed + n, device)[self._consumed:]
        self._consumed += n
        return flat.reshape(tuple(shape)).clone()


def get_lora_update_params(base_sigma: float, key_seed: int, rank: int, info: IterInfo, a: int,
                           b: int, noise_reuse: int, device=None):
    """eggroll.rs:86-103: returns (A (a,r) scaled by sign*base_sigma, B (b,r))."""
    A, B = ops.lora_factors(key_seed, info.epoch, noise_reuse, rank, a, b, base_sigma, 1,
                            first_thread=info.thread_id, device=device)
    return A[0], B[0]


def batched_lora_noise(base_sigma: float, key_seed: int, rank: int, tids: Sequence[int], epoch: int,
                       noise_reuse: int, a: int, b: int, device=None):
    """eggroll.rs:116-130: A (n,a,r) scaled, B (n,b,r); row i is bit-identical to
    get_lora_update_params for thread id tids[i]."""
    from .core import get_context
    dev = torch.device("cuda", get_context(device).device)
    t = torch.as_tensor(np.asarray(tids, dtype=np.int32), device=dev)
    return ops.lora_factors(key_seed, epoch, noise_reuse, rank, a, b, base_sigma, len(tids),
                            thread_ids=t, device=device)


def get_nonlora_update_params(base_sigma: float, key_seed: int, info: IterInfo,
                              shape: Tuple[int, int], noise_reuse: int, device=None) -> torch.Tensor:
    """eggroll.rs:312-324."""
    return ops.dense_noise(key_seed, info.epoch, noise_reuse, shape[0], shape[1], base_sigma, 1,
                           first_thread=info.thread_id, device=device)[0]


def convert_fitnesses_impl(group_size: int, raw: torch.Tensor) -> torch.Tensor:
    """noiser.rs:517-537."""
    return ops.convert_fitnesses(raw, group_size)


def combine_affine_grads(grad_acc: Sequence[torch.Tensor], ones_acc: Sequence[torch.Tensor],
                         mean: float, std: float, batch: int) -> List[torch.Tensor]:
    """eggroll.rs:902-915; pure scaling, done with the solver kernel's SGD form:
    out = g - o*mean, then scaled."""
    scale = float(np.float32(-1.0) / (np.float32(std) * np.sqrt(np.float32(batch))))
    out = []
    for g, o in zip(grad_acc, ones_acc):
        q = g.detach().clone().contiguous()
        ops.solver_step(ops.SGD, 0, q, o.contiguous(), lr=float(mean))  # q = g - o*mean
        z = torch.zeros_like(q)
        ops.solver_step(ops.SGD, 0, z, q, lr=-scale)                    # z = 0 - q*(-scale)
        out.append(z)
    return out


class LoraNoiseCache:
    """eggroll.rs:229-309.  One device-resident factor cache per LoRA parameter (None for the
    other classes), covering thread ids 0..batch-1.  The reference keeps (batch, a+b, r) in host
    memory and only allows noise_reuse == 0; here the caches live on the GPU, hold one entry per
    antithetic pair and are valid for the epoch bucket they were built for."""

    def __init__(self, buffers, shapes, batch: int, rank: int):
        self.buffers, self.shapes, self.batch, self.rank = buffers, shapes, batch, rank


def build_lora_noise_cache(params: Sequence[torch.Tensor], base_keys: Sequence[int],
                           es_classes: Sequence[int], batch: int, rank: int, noise_reuse: int,
                           epoch: int = 0) -> LoraNoiseCache:
    """eggroll.rs:275-309."""
    if batch % 2:
        raise ValueError("batch must consist of whole antithetic pairs")
    buffers = []
    for p, key, cls in zip(params, base_keys, es_classes):
        if cls != MM_PARAM:
            buffers.append(None)
            continue
        a, b = p.shape
        buffers.append(ops.FactorCache(key, epoch, noise_reuse, rank, a, b, batch // 2, 0, device=p.device))
    return LoraNoiseCache(buffers, [tuple(p.shape) for p in params], batch, rank)


def accumulated_update_cached(frozen: FrozenNoiserParams, noiser: NoiserParams,
                              params: Sequence[torch.Tensor], base_keys: Sequence[int],
                              es_classes: Sequence[int], conv_full: torch.Tensor,
                              thread_ids: Sequence[int], epoch: int, accumulate: int, chunk: int,
                              noise_cache: Optional[LoraNoiseCache] = None) -> List[torch.Tensor]:
    """eggroll.rs:579-702: the update of a batch of accumulate*chunk members computed chunk by
    chunk — per chunk sum_i f_i A_i B_i^T (A_i carrying sign*sigma/sqrt(rank)) is added to an
    accumulator, the total is scaled by -1/sqrt(batch), and the solver runs ONCE (its step
    counter advances by one, not by `accumulate`).  Thread ids must be first, first+1, ... with
    even `first` and even `chunk`, which is how the trainer numbers them."""
    if len(params) == 0:
        return []
    batch = accumulate * chunk
    tids = list(thread_ids)
    if len(tids) != batch or conv_full.numel() != batch:
        raise ValueError("thread_ids and conv_full must have accumulate*chunk entries")
    if chunk % 2 or tids[0] % 2 or any(t != tids[0] + i for i, t in enumerate(tids)):
        raise ValueError("thread ids must be consecutive, start even, and chunks must hold whole pairs")
    scale = float(np.float32(-1.0) / np.sqrt(np.float32(batch)))
    grads = []
    for idx, (p, key, cls) in enumerate(zip(params, base_keys, es_classes)):
        a, b = p.shape
        acc = torch.zeros((a, b), dtype=torch.float32, device=p.device)
        if cls == MM_PARAM:
            cache = noise_cache.buffers[idx] if noise_cache is not None else None
            for k in range(accumulate):
                lo = k * chunk
                ops.es_update(key, epoch, frozen.noise_reuse, frozen.rank, a, b, noiser.sigma,
                              conv_full[lo:lo + chunk].contiguous(), first_thread=tids[lo], out=acc,
                              cache=cache, mode=ops.UPDATE_RAW_ACC)
        elif cls == PARAM and not frozen.freeze_nonlora:
            for k in range(accumulate):
                lo = k * chunk
                # es_update_dense with n_total = chunk returns -sum_i f_i noise_i / sqrt(chunk)
                g = ops.es_update_dense(key, epoch, frozen.noise_reuse, (a, b), noiser.sigma,
                                        conv_full[lo:lo + chunk].contiguous(), first_thread=tids[lo],
                                        n_total=chunk)
                ops.solver_step(ops.SGD, 0, acc, g, lr=float(np.sqrt(np.float32(chunk))))  # acc -= sqrt(chunk)*g
        g = torch.zeros_like(acc)
        ops.solver_step(ops.SGD, 0, g, acc, lr=-scale)  # g = scale * acc
        grads.append(g)
    return frozen.solver.update(params, grads, noiser.opt_state)


def accumulated_update(frozen, noiser, params, base_keys, es_classes, conv_full, thread_ids, epoch,
                       accumulate, chunk) -> List[torch.Tensor]:
    """eggroll.rs:550-575: the uncached form (factors regenerated chunk by chunk)."""
    return accumulated_update_cached(frozen, noiser, params, base_keys, es_classes, conv_full,
                                     thread_ids, epoch, accumulate, chunk, None)


def _dense_fitness(scores: np.ndarray, iterinfos: Sequence[IterInfo], noise_reuse: int
                   ) -> Dict[int, Tuple[int, np.ndarray]]:
    """Scatter per-member scores into dense, pair-aligned vectors keyed by epoch bucket."""
    groups: Dict[int, Dict[int, float]] = {}
    for s, info in zip(scores, iterinfos):
        te = 0 if noise_reuse == 0 else int(info.epoch / noise_reuse)
        if info.thread_id < 0:
            raise ValueError("thread ids must be non-negative")
        groups.setdefault(te, {})
        groups[te][info.thread_id] = groups[te].get(info.thread_id, 0.0) + float(s)
    out = {}
    for te, d in groups.items():
        lo = min(d) // 2 * 2
        hi = max(d) // 2 * 2 + 2
        vec = np.zeros(hi - lo, dtype=np.float32)
        for tid, s in d.items():
            vec[tid - lo] = np.float32(s)
        out[te] = (lo, vec)
    return out


class EggRoll:
    """The EggRoll noiser (eggroll.rs:917-1005)."""

    #: AltEggRoll sets this: its LoRA update contracts the signs of the factors.
    sign_factors = False

    def do_mm(self, frozen: FrozenNoiserParams, noiser: NoiserParams, param: torch.Tensor,
              base_key: int, iterinfo: Optional[IterInfo], x: torch.Tensor) -> torch.Tensor:
        """x (bm, b) @ param.T (+ LoRA noise of this member); eggroll.rs:419-446."""
        bm = x.shape[0]
        if iterinfo is None:
            return ops.perturbed_linear(x, param, n_pop=1, bm=bm, perturb=False)
        return ops.perturbed_linear(x, param, n_pop=1, bm=bm, sigma=noiser.sigma, rank=frozen.rank,
                                    key=base_key, epoch=iterinfo.epoch,
                                    first_thread=iterinfo.thread_id, noise_reuse=frozen.noise_reuse)

    def do_mm_population(self, frozen: FrozenNoiserParams, noiser: NoiserParams, param: torch.Tensor,
                         base_key: int, epoch: int, first_thread: int, x: torch.Tensor,
                         t_steps: int = 1, **kw) -> torch.Tensor:
        """All members at once: x is (t_steps, n_pop, bm, k); member i has thread id
        first_thread + i.  Row-for-row equal to calling do_mm per member."""
        n_pop, bm = x.shape[-3], x.shape[-2]
        return ops.perturbed_linear(x, param, n_pop=n_pop, bm=bm, t_steps=t_steps,
                                    sigma=noiser.sigma, rank=frozen.rank, key=base_key, epoch=epoch,
                                    first_thread=first_thread, noise_reuse=frozen.noise_reuse, **kw)

    def do_Tmm(self, frozen, noiser, param, base_key, iterinfo, x):  # noqa: N802
        """x @ param (+ x·A·Bᵀ); eggroll.rs:450-477.  Not on the accelerated path: the base
        product uses the clean linear kernel on paramᵀ and the rank-r term is assembled from
        the materialised factors."""
        pt = param.t().contiguous()
        base = ops.perturbed_linear(x, pt, n_pop=1, bm=x.shape[0], perturb=False)
        if iterinfo is None:
            return base
        a, b = param.shape
        A, B = get_lora_update_params(ops.base_sigma(noiser.sigma, frozen.rank), base_key,
                                      frozen.rank, iterinfo, a, b, frozen.noise_reuse, x.device)
        t = ops.perturbed_linear(x, A.t().contiguous(), n_pop=1, bm=x.shape[0], perturb=False)
        u = ops.perturbed_linear(t, B.contiguous(), n_pop=1, bm=x.shape[0], perturb=False)
        out = base.clone()
        ops.solver_step(ops.SGD, 0, out, u, lr=-1.0)  # out = base - u*(-1)
        return out

    def do_emb(self, *args, **kwargs):
        """eggroll.rs:943-954 leaves this unimplemented as well."""
        raise NotImplementedError("EggRoll.do_emb is unimplemented in the reference")

    def get_noisy_standard(self, frozen, noiser, param, base_key, iterinfo):
        """eggroll.rs:480-503."""
        if iterinfo is None or frozen.freeze_nonlora:
            return param.clone()
        noise = get_nonlora_update_params(noiser.sigma, base_key, iterinfo, tuple(param.shape),
                                          frozen.noise_reuse, param.device)
        out = param.detach().clone().contiguous()
        ops.solver_step(ops.SGD, 0, out, noise.contiguous(), lr=-1.0)  # param + noise
        return out

    def convert_fitnesses(self, frozen: FrozenNoiserParams, noiser: NoiserParams,
                          raw: torch.Tensor) -> torch.Tensor:
        """eggroll.rs:967-992."""
        return ops.convert_fitnesses(raw, frozen.group_size)

    def grads(self, frozen: FrozenNoiserParams, noiser: NoiserParams, params: Sequence[torch.Tensor],
              base_keys: Sequence[int], fitnesses: torch.Tensor, iterinfos: Sequence[IterInfo],
              es_classes: Sequence[int]) -> List[torch.Tensor]:
        """The per-parameter `-g*sqrt(N)` of do_update_with (eggroll.rs:384-404)."""
        n_total = len(iterinfos)
        infos = list(iterinfos)
        contiguous = (n_total % 2 == 0 and infos[0].thread_id % 2 == 0 and all(
            infos[i].thread_id == infos[0].thread_id + i and infos[i].epoch == infos[0].epoch
            for i in range(n_total)))
        if contiguous:
            groups = {None: (infos[0].thread_id, fitnesses, infos[0].epoch)}
        else:
            dense = _dense_fitness(fitnesses.detach().cpu().numpy(), infos, frozen.noise_reuse)
            nr = max(frozen.noise_reuse, 1)
            groups = {te: (lo, torch.as_tensor(vec, device=fitnesses.device), te * nr)
                      for te, (lo, vec) in dense.items()}
        out = []
        for p, key, cls in zip(params, base_keys, es_classes):
            a, b = p.shape
            total = None
            for lo, vec, ep in groups.values():
                if cls == MM_PARAM:
                    g = ops.es_update(key, ep, frozen.noise_reuse, frozen.rank, a, b, noiser.sigma,
                                      vec, first_thread=lo, n_total=n_total,
                                      sign_factors=self.sign_factors)
                elif cls == PARAM and not frozen.freeze_nonlora:
                    g = ops.es_update_dense(key, ep, frozen.noise_reuse, (a, b), noiser.sigma, vec,
                                            first_thread=lo, n_total=n_total)
                else:
                    g = torch.zeros((a, b), dtype=torch.float32, device=p.device)
                if total is None:
                    total = g
                else:
                    ops.solver_step(ops.SGD, 0, total, g, lr=-1.0)  # total += g
            out.append(total)
        return out

    def do_updates(self, frozen: FrozenNoiserParams, noiser: NoiserParams,
                   params: Sequence[torch.Tensor], base_keys: Sequence[int], fitnesses: torch.Tensor,
                   iterinfos: Sequence[IterInfo], es_classes: Sequence[int]) -> List[torch.Tensor]:
        """eggroll.rs:994-1005 / do_updates_impl 508-528: returns the updated parameters and
        advances noiser.opt_state."""
        if len(params) == 0:
            return []
        grads = self.grads(frozen, noiser, params, base_keys, fitnesses, iterinfos, es_classes)
        return frozen.solver.update(params, grads, noiser.opt_state)


class AltEggRoll(EggRoll):
    """hyperscalees-noiser/src/alteggroll.rs: EggRoll everywhere except the LoRA update, which
    uses sign(A_i) * (sigma * f_i / sqrt(rank)) and sign(B_i) (alteggroll.rs:65-90)."""

    sign_factors = True


class EggRollBS(EggRoll):
    """hyperscalees-noiser/src/eggroll_bs.rs: EggRoll with baseline subtraction, a member mask
    and a trust-region clipped solver.

    * noise of thread ids with `tid % group_size < 2` is zero (eggroll_bs.rs:73-125): such a
      member's forward is the clean product and it contributes nothing to the update;
    * convert_fitnesses turns the (Q, G) raw scores into G per-direction values (226-250);
    * init_noiser wraps the solver in clip_by_global_norm (37-65)."""

    @staticmethod
    def init_noiser(params, sigma: float, _lr: float, group_size: int, freeze_nonlora: bool,
                    noise_reuse: int, rank: int, trust_region_norm: float, solver: Solver):
        return init_noiser(params, sigma, _lr, group_size, freeze_nonlora, noise_reuse, rank,
                           Solver.trust_region(trust_region_norm, solver))

    @staticmethod
    def mask(info: IterInfo, group_size: int) -> float:
        """eggroll_bs.rs:73-80."""
        return 1.0 if group_size > 0 and info.thread_id % group_size >= 2 else 0.0

    def do_mm(self, frozen, noiser, param, base_key, iterinfo, x):
        if iterinfo is not None and self.mask(iterinfo, frozen.group_size) == 0.0:
            iterinfo = None   # both factors are multiplied by the mask: the rank-r term vanishes
        return super().do_mm(frozen, noiser, param, base_key, iterinfo, x)

    def do_Tmm(self, frozen, noiser, param, base_key, iterinfo, x):  # noqa: N802
        if iterinfo is not None and self.mask(iterinfo, frozen.group_size) == 0.0:
            iterinfo = None
        return super().do_Tmm(frozen, noiser, param, base_key, iterinfo, x)

    def get_noisy_standard(self, frozen, noiser, param, base_key, iterinfo):
        if iterinfo is not None and self.mask(iterinfo, frozen.group_size) == 0.0:
            return param.clone()
        return super().get_noisy_standard(frozen, noiser, param, base_key, iterinfo)

    def convert_fitnesses(self, frozen: FrozenNoiserParams, noiser: NoiserParams,
                          raw: torch.Tensor) -> torch.Tensor:
        return ops.convert_fitnesses_bs(raw, frozen.group_size)

    def grads(self, frozen, noiser, params, base_keys, fitnesses, iterinfos, es_classes):
        """do_update (eggroll_bs.rs:198-224): EggRoll's update with every member's factors
        multiplied by its mask, i.e. with masked fitnesses."""
        infos = list(iterinfos)
        m = torch.as_tensor(np.asarray([self.mask(i, frozen.group_size) for i in infos], dtype=np.float32),
                            device=fitnesses.device)
        return super().grads(frozen, noiser, params, base_keys, ops.vector_mul(fitnesses.contiguous(), m),
                             infos, es_classes)
