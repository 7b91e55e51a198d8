"""Host-side mirror of hyperscalees-models/src/snn_transformer.rs: the SNN-rate
transformer classifier whose `forward_batched` runs a whole chunk of population
members per call.

Every matrix product goes through `hses_perturbed_linear` (a member's rank-r
noise is regenerated from `(base key, epoch, thread id)`, bit-identical to the
`batched_lora_noise` tensors the reference trainer builds,
hyperscalees/src/bin/snn_transformer_train.rs:401-418), the attention core
through `hses_spiking_attention` mode 2 with one beta per member, the rate code
through `hses_rate_encode`.  Adds, the swish gate and the token mean are plain
tensor arithmetic.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import ops
from .noiser import EMB_PARAM, MM_PARAM, PARAM


@dataclass
class TrainNoise:
    """TrainNoise, snn_transformer.rs:35-52, with the LoRA tensors replaced by what they are
    generated from: `sigma`, `rank`, one base key per parameter index, epoch and the thread id
    of the chunk's first member (members of a chunk have consecutive ids).  The dense
    per-member noises are explicit tensors as in the reference (its trainer draws them from an
    unseeded generator)."""
    sigma: float
    rank: int
    base_keys: Sequence[int]
    epoch: int = 0
    first_thread: int = 0
    noise_reuse: int = 0
    mm_indices: Optional[Sequence[int]] = None      # None = every MM parameter
    caches: Optional[dict] = None                   # parameter index -> ops.FactorCache (see build_caches)
    pos_emb: Optional[torch.Tensor] = None          # (n, num_tokens, d_model)
    out_gain: Optional[torch.Tensor] = None         # (n, 1)
    beta: Optional[torch.Tensor] = None             # (n, 1)


class SnnTransformer:
    """SnnTransformer::new / params / es_map / forward_batched (snn_transformer.rs:118-413)."""

    def __init__(self, token_in_dim: int, num_tokens: int, num_classes: int, d_model: int, num_heads: int,
                 num_blocks: int, device=None, seed: int = 0):
        from .core import default_device
        if d_model % num_heads:
            raise ValueError(f"d_model({d_model}) must be a multiple of num_heads({num_heads})")
        self.device = torch.device(device) if device is not None else default_device()
        g = np.random.Generator(np.random.PCG64(seed))

        def mm(n_in: int, n_out: int) -> torch.Tensor:
            # Mm::new(in, out): weight (out, in), N(0, 1/sqrt(in)) (common.rs:113-121)
            w = g.standard_normal((n_out, n_in)).astype(np.float32) / np.float32(np.sqrt(n_in))
            return torch.as_tensor(w, device=self.device)

        head_dim = d_model // num_heads
        self.in_q, self.in_k, self.in_v = mm(token_in_dim, d_model), mm(token_in_dim, d_model), mm(token_in_dim, d_model)
        self.pos_emb = torch.zeros(num_tokens, d_model, device=self.device)
        self.blocks = []
        for _ in range(num_blocks):
            self.blocks.append({
                "q": [mm(d_model, head_dim) for _ in range(num_heads)],
                "k": [mm(d_model, head_dim) for _ in range(num_heads)],
                "v": [mm(d_model, head_dim) for _ in range(num_heads)],
                "o": mm(d_model, d_model), "ff1": mm(d_model, d_model), "ff2": mm(d_model, d_model)})
        self.out = mm(d_model, num_classes)
        self.out_gain = torch.ones(1, device=self.device)
        raw_beta = float(np.log(np.exp(np.float32(1.0) / np.sqrt(np.float32(head_dim))) - 1.0))
        self.beta = torch.full((1,), raw_beta, device=self.device)
        self.tau_m, self.proj_gain, self.g_inh, self.tau_a, self.n_iter = 20.0, 2.0, 0.5, 5.0, 8
        self.num_heads, self.num_tokens, self.token_in_dim = num_heads, num_tokens, token_in_dim
        self.d_model, self.head_dim = d_model, head_dim

    # ---- parameter plumbing (snn_transformer.rs:204-253) ----
    def params(self) -> List[torch.Tensor]:
        ps = [self.in_q, self.in_k, self.in_v, self.pos_emb]
        for blk in self.blocks:
            ps += blk["q"] + blk["k"] + blk["v"] + [blk["o"], blk["ff1"], blk["ff2"]]
        ps += [self.out, self.out_gain.view(1, 1), self.beta.view(1, 1)]
        return ps

    def es_map(self) -> List[int]:
        total = 3 + 1 + len(self.blocks) * (3 * self.num_heads + 3) + 1 + 2
        m = [MM_PARAM] * total
        m[3] = EMB_PARAM
        m[total - 1] = PARAM
        m[total - 2] = PARAM
        return m

    def block_base(self, b: int) -> int:
        return 4 + b * (3 * self.num_heads + 3)

    def out_param_index(self) -> int:
        return 4 + len(self.blocks) * (3 * self.num_heads + 3)

    # ---- nn, snn_transformer.rs:273-297 ----
    def nn(self, idx: int, x: torch.Tensor, w: torch.Tensor, noise: Optional[TrainNoise],
           out: Optional[torch.Tensor] = None, t_steps: int = 1) -> torch.Tensor:
        """x (t_steps, n, tokens, in) or (n, tokens, in); w (out, in) -> same leading dims with out
        columns.  Member j of the chunk owns rows [j*tokens, (j+1)*tokens) of every step."""
        n, tokens = x.shape[-3], x.shape[-2]
        perturb = noise is not None and (noise.mm_indices is None or idx in noise.mm_indices)
        kw = {}
        if perturb:
            kw = dict(sigma=noise.sigma, rank=noise.rank, key=noise.base_keys[idx], epoch=noise.epoch,
                      first_thread=noise.first_thread, noise_reuse=noise.noise_reuse)
            if noise.caches is not None and idx in noise.caches:
                kw["cache"] = noise.caches[idx]
        y = ops.perturbed_linear(x, w, n_pop=n, bm=tokens, t_steps=t_steps, perturb=perturb, out=out, **kw)
        return y

    def build_caches(self, noise: TrainNoise, n: int) -> dict:
        """The chunk's factors of every MM parameter, generated once (what the reference trainer does
        with `batched_lora_noise` before the forward and the gradient einsum of a chunk,
        snn_transformer_train.rs:401-418).  Assign the result to `noise.caches`."""
        if n % 2 or noise.first_thread % 2:
            raise ValueError("a cache covers whole antithetic pairs: n and first_thread must be even")
        caches = {}
        for idx, (p, cls) in enumerate(zip(self.params(), self.es_map())):
            if cls != MM_PARAM or (noise.mm_indices is not None and idx not in noise.mm_indices):
                continue
            a, b = p.shape
            caches[idx] = ops.FactorCache(noise.base_keys[idx], noise.epoch, noise.noise_reuse, noise.rank, a, b,
                                          n // 2, first_pair=noise.first_thread // 2, device=self.device)
        return caches

    # ---- encode, snn_transformer.rs:305-339 ----
    def encode(self, x: torch.Tensor, noise: Optional[TrainNoise]) -> torch.Tensor:
        T, n, in_dim = x.shape
        nt, tin, d = self.num_tokens, self.token_in_dim, self.d_model
        xt = x.reshape(T, n, nt, tin)
        rates = []
        for idx, w in ((0, self.in_q), (1, self.in_k), (2, self.in_v)):
            proj = self.nn(idx, xt, w, noise, t_steps=T)                 # (T*n*nt, d): every step in one launch
            mean = ops.time_mean(proj.view(T, n * nt, d))                # sum over steps times 1/T
            rates.append(ops.rate_encode(mean, self.proj_gain))
        return ((rates[0] + rates[1] + rates[2]) / 3.0).view(n, nt, d)

    # ---- forward_batched, snn_transformer.rs:345-413 ----
    def forward_batched(self, x: torch.Tensor, noise: Optional[TrainNoise] = None) -> torch.Tensor:
        T, n, in_dim = x.shape
        if in_dim != self.num_tokens * self.token_in_dim:
            raise ValueError(f"input width must be num_tokens*token_in_dim = {self.num_tokens * self.token_in_dim}, "
                             f"got {in_dim}")
        nt, d, H, hd = self.num_tokens, self.d_model, self.num_heads, self.head_dim
        xh = self.encode(x.contiguous(), noise) + self.pos_emb.unsqueeze(0)
        if noise is not None and noise.pos_emb is not None:
            xh = xh + noise.pos_emb
        beta_raw = self.beta.view(1, 1)
        if noise is not None and noise.beta is not None:
            beta_raw = beta_raw + noise.beta                              # (n, 1)
        beta = torch.log1p(torch.exp(beta_raw)).expand(n, 1).contiguous().view(n)   # softplus, one per member
        qb = torch.empty(n, nt, d, device=x.device)
        kb, vb = torch.empty_like(qb), torch.empty_like(qb)
        for b, blk in enumerate(self.blocks):
            base = self.block_base(b)
            xh = xh.contiguous()
            for h in range(H):
                # head h's projections land in columns [h*hd, (h+1)*hd) of the shared buffers,
                # which is the layout the attention kernel reads and the concat the reference builds
                sl = slice(h * hd, (h + 1) * hd)
                self.nn(base + 3 * h, xh, blk["q"][h], noise, out=qb.view(n * nt, d)[:, sl])
                self.nn(base + 3 * h + 1, xh, blk["k"][h], noise, out=kb.view(n * nt, d)[:, sl])
                self.nn(base + 3 * h + 2, xh, blk["v"][h], noise, out=vb.view(n * nt, d)[:, sl])
            concat = ops.spiking_attention(qb, kb, vb, H, mode=2, tau_m=self.tau_a, g_inh=self.g_inh,
                                           n_iter=self.n_iter, beta_per_seq=beta)
            attn = self.nn(base + 3 * H, concat, blk["o"], noise).view(n, nt, d)
            xh = (xh + attn).contiguous()
            ff1 = self.nn(base + 3 * H + 1, xh, blk["ff1"], noise).view(n, nt, d)
            act = ff1 * torch.sigmoid(ff1)
            ff2 = self.nn(base + 3 * H + 2, act, blk["ff2"], noise).view(n, nt, d)
            xh = xh + ff2
        pooled = xh.mean(dim=1).contiguous()                              # (n, d_model)
        logits = self.nn(self.out_param_index(), pooled.view(n, 1, d), self.out, noise)
        gain = self.out_gain.view(1, 1)
        if noise is not None and noise.out_gain is not None:
            gain = gain + noise.out_gain
        return logits * gain
