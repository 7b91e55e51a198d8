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
