"""Token-level spiking self-attention transformer: the language-model form of the spiking
transformer (uniform token ids in, next-token log-likelihood out).

The reference has the parts, not this composition: the block structure (per-head Q/K/V
projections, output projection, residual, feed-forward, residual) is
hyperscalees-models/src/snn_transformer.rs:345-413; Q/K/V as LIF firing rates over T steps
are src/hyperscalees/models/snn_self_attention.py:114-131; the embedding hook `do_emb` is
declared and left unimplemented in both noisers (src/hyperscalees/noiser/eggroll.py:93,
hyperscalees-noiser/src/eggroll.rs:943-954).  What is fixed here beyond them: the embedding is
the clean gather plus the member's rank-r term on the gathered row, the Q/K/V currents are
constant over the T LIF steps (token embeddings do not change in time), the attention core
is the spike product without softmax under a causal mask, the feed-forward widens by
`mlp_ratio`, and the fitness is the mean next-token log-likelihood.  Parity is pinned
against a numpy composition of the CPU restatement's pieces (oracle/spiking_lm.py), not
against a reference output: none exists for this model.

Every matrix product is one `hses_perturbed_linear` launch over the chunk of members, with
each member's rank-r noise regenerated from (base key, epoch, thread id).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import ops
from .noiser import EMB_PARAM, MM_PARAM, PARAM


@dataclass
class LmNoise:
    """What a chunk's perturbation is generated from: sigma, rank, one base key per parameter
    index, the epoch and the thread id of the chunk's first member (consecutive ids)."""
    sigma: float
    rank: int
    base_keys: Sequence[int]
    epoch: int = 0
    first_thread: int = 0
    noise_reuse: int = 0


class SpikingLM:
    def __init__(self, vocab: int, seq_len: int, d_model: int, num_heads: int, num_blocks: int,
                 mlp_ratio: int = 4, T: int = 4, tau_m: float = 2.0, v_th: float = 0.3, device=None, seed: int = 0):
        from .core import default_device
        if d_model % num_heads or d_model % 4:
            raise ValueError("d_model must be a multiple of num_heads and of 4")
        self.device = torch.device(device) if device is not None else default_device()
        g = np.random.Generator(np.random.PCG64(seed))

        def mm(n_in: int, n_out: int) -> torch.Tensor:
            # Mm::new(in, out): weight (out, in), N(0, 1/sqrt(in)) (common.rs:113-121)
            w = g.standard_normal((n_out, n_in)).astype(np.float32) / np.float32(np.sqrt(n_in))
            return torch.as_tensor(w, device=self.device)

        hd = d_model // num_heads
        # Embedding::new(in = vocab, out = d): (vocab, d), N(0, 1/sqrt(vocab)) (common.py:111-119)
        self.emb = torch.as_tensor(g.standard_normal((vocab, d_model)).astype(np.float32) / np.float32(np.sqrt(vocab)),
                                   device=self.device)
        self.pos_emb = torch.as_tensor(g.standard_normal((seq_len, d_model)).astype(np.float32) * np.float32(0.02),
                                       device=self.device)
        self.blocks = []
        for _ in range(num_blocks):
            self.blocks.append({
                "q": [mm(d_model, hd) for _ in range(num_heads)],
                "k": [mm(d_model, hd) for _ in range(num_heads)],
                "v": [mm(d_model, hd) for _ in range(num_heads)],
                "o": mm(d_model, d_model), "ff1": mm(d_model, mlp_ratio * d_model),
                "ff2": mm(mlp_ratio * d_model, d_model)})
        self.out = mm(d_model, vocab)
        self.out_gain = 1.0
        self.beta = float(1.0 / np.sqrt(np.float32(hd)))
        self.vocab, self.seq_len, self.d_model, self.num_heads, self.head_dim = vocab, seq_len, d_model, num_heads, hd
        self.T, self.tau_m, self.v_th = T, tau_m, v_th

    # ---- parameter plumbing, in the order of snn_transformer.rs:204-253 ----
    def params(self) -> List[torch.Tensor]:
        ps = [self.emb, self.pos_emb]
        for blk in self.blocks:
            ps += blk["q"] + blk["k"] + blk["v"] + [blk["o"], blk["ff1"], blk["ff2"]]
        ps += [self.out]
        return ps

    def es_map(self) -> List[int]:
        m = [MM_PARAM] * len(self.params())
        m[0] = EMB_PARAM
        m[1] = PARAM          # position rows: a dense leaf, carried clean by forward_population
        return m

    def block_base(self, b: int) -> int:
        return 2 + b * (3 * self.num_heads + 3)

    def out_param_index(self) -> int:
        return 2 + len(self.blocks) * (3 * self.num_heads + 3)

    def nn(self, idx: int, x: torch.Tensor, w: torch.Tensor, n: int, rows_per_member: int,
           noise: Optional[LmNoise], out: Optional[torch.Tensor] = None, same_x: bool = False) -> torch.Tensor:
        """same_x: the call right before this one projected the same x with a matrix of the same shape (the
        per-head Q/K/V of a block): the tensor-core path keeps that call's fp16 operand split of x."""
        kw = {}
        if noise is not None:
            kw = dict(sigma=noise.sigma, rank=noise.rank, key=noise.base_keys[idx], epoch=noise.epoch,
                      first_thread=noise.first_thread, noise_reuse=noise.noise_reuse)
            if noise.first_thread % 2 == 0 and n % 2 == 0:
                # A member owns thousands of rows here and its factors a few hundred values: they are
                # generated once per call into a factor cache (same bits as regenerating them in the
                # kernels), which lets narrow layers take the tensor-core path as well
                a, k = w.shape
                kw["cache"] = ops.FactorCache(noise.base_keys[idx], noise.epoch, noise.noise_reuse, noise.rank, a, k,
                                              n // 2, first_pair=noise.first_thread // 2, device=self.device)
        return ops.perturbed_linear(x, w, n_pop=n, bm=rows_per_member, perturb=noise is not None, out=out,
                                    reuse_x_split=same_x, **kw)

    def nn_heads(self, idxs, x: torch.Tensor, ws, n: int, rows_per_member: int, noise: Optional[LmNoise],
                 out: torch.Tensor, same_x: bool) -> bool:
        """The per-head projections `ws` (parameters idxs) of one x in ONE call: the heads' matrices stacked
        along the rows, every head with its own noise, columns [h*hd, (h+1)*hd) of `out` for head h.  x is
        read once instead of once per head.  Returns False when the shapes do not allow it (the caller then
        projects head by head)."""
        hd = ws[0].shape[0]
        if noise is None:
            ops.perturbed_linear(x, torch.cat(list(ws), 0), n_pop=n, bm=rows_per_member, perturb=False, out=out,
                                 reuse_x_split=same_x)
            return True
        groupable = (noise.first_thread % 2 == 0 and n % 2 == 0 and noise.rank in (1, 2, 3, 4, 8, 16) and
                     (hd % 32 == 0 or (hd % 16 == 0 and noise.rank >= 8)))
        if not groupable:
            return False
        k = ws[0].shape[1]
        caches = [ops.FactorCache(noise.base_keys[i], noise.epoch, noise.noise_reuse, noise.rank, hd, k, n // 2,
                                  first_pair=noise.first_thread // 2, device=self.device) for i in idxs]
        grouped = ops.GroupedFactorCache(caches)
        ops.perturbed_linear(x, torch.cat(list(ws), 0), n_pop=n, bm=rows_per_member, sigma=noise.sigma,
                             rank=noise.rank, key=grouped.key, epoch=noise.epoch, first_thread=noise.first_thread,
                             noise_reuse=noise.noise_reuse, cache=grouped, n_groups=len(ws), out=out,
                             reuse_x_split=same_x)
        return True

    def forward_population(self, ids: torch.Tensor, noise: Optional[LmNoise] = None) -> torch.Tensor:
        """ids (n, seqs, L) int32: member j evaluates its own `seqs` sequences -> logits
        (n*seqs*L, vocab), before the output gain."""
        n, seqs, L = ids.shape
        if L != self.seq_len:
            raise ValueError(f"sequences must be {self.seq_len} tokens long")
        d, H, hd = self.d_model, self.num_heads, self.head_dim
        rpm = seqs * L
        rows = n * rpm
        flat = ids.reshape(rows).contiguous()
        A = B = None
        if noise is not None:
            A, B = ops.lora_factors(noise.base_keys[0], noise.epoch, noise.noise_reuse, noise.rank, self.vocab, d,
                                    ops.base_sigma(noise.sigma, noise.rank), n, first_thread=noise.first_thread,
                                    device=self.device)
        x = ops.embedding(flat, self.emb, self.pos_emb, A, B, rows_per_member=rpm)
        del A, B
        qc = torch.empty(rows, d, device=self.device)
        kc, vc = torch.empty_like(qc), torch.empty_like(qc)
        beta = torch.full((n * seqs,), self.beta, device=self.device)
        for b, blk in enumerate(self.blocks):
            base = self.block_base(b)
            # head h's currents land in columns [h*hd, (h+1)*hd): the layout the attention kernel reads.
            # The heads of Q, of K and of V go out as three grouped calls (x read three times instead of
            # twelve, split into tensor-core operands once); head by head where the shapes do not allow it
            grouped = True
            for j, (name, buf) in enumerate((("q", qc), ("k", kc), ("v", vc))):
                grouped = grouped and self.nn_heads([base + 3 * h + j for h in range(H)], x, blk[name], n, rpm, noise,
                                                    buf, same_x=j > 0)
            if not grouped:
                for h in range(H):
                    sl = slice(h * hd, (h + 1) * hd)
                    self.nn(base + 3 * h, x, blk["q"][h], n, rpm, noise, out=qc[:, sl], same_x=h > 0)
                    self.nn(base + 3 * h + 1, x, blk["k"][h], n, rpm, noise, out=kc[:, sl], same_x=True)
                    self.nn(base + 3 * h + 2, x, blk["v"][h], n, rpm, noise, out=vc[:, sl], same_x=True)
            # LIF over T steps on the constant currents, firing rates in place
            for buf in (qc, kc, vc):
                ops.lif_rate(buf, self.T, self.tau_m, self.v_th, out=buf)
            attn = ops.spiking_attention(qc.view(n * seqs, L, d), kc.view(n * seqs, L, d), vc.view(n * seqs, L, d), H,
                                         mode=3, beta_per_seq=beta)
            ops.add_inplace(x, self.nn(base + 3 * H, attn.view(rows, d), blk["o"], n, rpm, noise))
            ff1 = self.nn(base + 3 * H + 1, x, blk["ff1"], n, rpm, noise)
            ops.swish(ff1, out=ff1)
            ops.add_inplace(x, self.nn(base + 3 * H + 2, ff1, blk["ff2"], n, rpm, noise))
            del attn, ff1
        return self.nn(self.out_param_index(), x, self.out, n, rpm, noise)

    def fitness(self, ids: torch.Tensor, noise: Optional[LmNoise] = None, chunk_members: int = 1024) -> torch.Tensor:
        """Mean next-token log-likelihood per member; the population is walked in chunks of whole
        antithetic pairs so that the activations of one chunk (not of all members) are alive."""
        n, seqs, L = ids.shape
        out = torch.empty(n, dtype=torch.float32, device=self.device)
        chunk_members = max(2, chunk_members - chunk_members % 2)
        for lo in range(0, n, chunk_members):
            hi = min(n, lo + chunk_members)
            nz = None
            if noise is not None:
                nz = LmNoise(noise.sigma, noise.rank, noise.base_keys, noise.epoch, noise.first_thread + lo,
                             noise.noise_reuse)
            part = ids[lo:hi].contiguous()
            logits = self.forward_population(part, nz)
            out[lo:hi] = ops.token_fitness(logits, part.reshape(-1), hi - lo, seqs, L, gain=self.out_gain)
            del logits
        return out
