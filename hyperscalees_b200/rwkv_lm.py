"""RWKV-7 language model evaluated by a whole EggRoll population: embedding -> ln0 -> n_layer x
(ln1 -> TimeMixing -> ln2 -> ChannelMixing) -> ln_out -> head, one sequence per member, fitness =
mean next-token log-likelihood.

Stack and data flow follow src/hyperscalees/models/llm/rwkv7.py:222-253 (`forward_seq`) and
llm/llm.py:91-104 (`_forward`); the block algebra is hyperscalees-models/src/llm.rs:348-479
(`TimeMixing::forward`, with tanh on the v1 and a1 stages as written there) and 192-213
(`ChannelMixing::forward`).  As in `get_es_map` (rwkv7.py:160-179) every Linear and TMM weight of
the blocks carries the member's low-rank noise (do_mm / do_Tmm), the embedding and the head are
excluded, and the vectors and norms are dense leaves; they are evaluated clean here (the
`freeze_nonlora` setting of the noiser).  Weights are bf16 values held in fp32 tensors; products
round their operands to bf16 and accumulate in fp32 (`precision = BF16`), state and everything
between the products is fp32.

The members' sequences are laid end to end as rows (member j owns rows [j*T, (j+1)*T)); every
member starts from a zero state, so the token shift sees a `new_starts` mark on each member's
first row and the recurrence runs as one (member, head) problem per warp.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import ops

VECTORS = ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g", "w0", "v0", "a0", "k_k", "k_a")
LINEAR = ("receptance", "key", "value", "output")          # (out, in), do_mm
TMM_1 = ("w1", "v1", "a1", "g1")                            # (in = C, out = lora dim), do_Tmm
TMM_2 = ("w2", "v2", "a2", "g2")                            # (in = lora dim, out = C), do_Tmm


def bf16_round(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


@dataclass
class LmNoise:
    sigma: float
    rank: int
    epoch: int = 0
    first_thread: int = 0
    noise_reuse: int = 0


class RwkvLM:
    def __init__(self, n_layer: int, d_model: int, vocab: int, head_size: int = 64, ffn_mult: int = 4,
                 lora_dims: Sequence[int] = (64, 32, 64, 128), device=None, seed: int = 0, std: float = 0.02):
        from .core import default_device
        if d_model % head_size:
            raise ValueError("d_model must be a multiple of head_size")
        self.device = torch.device(device) if device is not None else default_device()
        self.n_layer, self.C, self.vocab, self.S, self.H = n_layer, d_model, vocab, head_size, d_model // head_size
        g = torch.Generator(device="cpu").manual_seed(seed)
        C = d_model

        def mat(*shape, s=std):
            return bf16_round(torch.randn(*shape, generator=g) * s).to(self.device).contiguous()

        def vec(n, lo=0.0, hi=1.0):
            return bf16_round(torch.rand(n, generator=g) * (hi - lo) + lo).to(self.device)

        self.emb = mat(vocab, C)
        self.vocab_pad = (vocab + 127) // 128 * 128          # the head's rows padded to a column tile
        head = torch.zeros(self.vocab_pad, C)
        head[:vocab] = bf16_round(torch.randn(vocab, C, generator=g) * std)
        self.head = head.to(self.device).contiguous()
        ones, zeros = torch.ones(C, device=self.device), torch.zeros(C, device=self.device)
        self.ln0 = (ones.clone(), zeros.clone())
        self.ln_out = (ones.clone(), zeros.clone())
        dw, dv, da, dg = lora_dims
        dims = {"w1": dw, "v1": dv, "a1": da, "g1": dg}
        self.layers: List[Dict[str, torch.Tensor]] = []
        for _ in range(n_layer):
            w = {n: vec(C) for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g")}
            w.update({n: vec(C, -0.5, 0.5) for n in ("w0", "v0", "a0")})
            w.update({"k_k": vec(C, 0.5, 1.5), "k_a": vec(C, 0.5, 1.5), "r_k": vec(C, -0.3, 0.3).view(self.H, self.S)})
            for n in LINEAR:
                w[n] = mat(C, C)
            for n1, n2 in zip(TMM_1, TMM_2):
                # kept transposed, (out, in): the layout hses_perturbed_linear takes; the reference
                # stores (in, out) and its factor block follows that shape (factor_order = 1)
                w[n1] = mat(dims[n1], C)
                w[n2] = mat(C, dims[n1])
            w["ln_x"] = (ones.clone(), zeros.clone())
            w["ln1"] = (ones.clone(), zeros.clone())
            w["ln2"] = (ones.clone(), zeros.clone())
            w["ffn_x_k"] = vec(C)
            w["ffn_key"] = mat(ffn_mult * C, C)
            w["ffn_value"] = mat(C, ffn_mult * C)
            self.layers.append(w)
        # one base key per noised matrix, numbered through the layers in a fixed order
        self.matrix_names = list(LINEAR) + list(TMM_1) + list(TMM_2) + ["ffn_key", "ffn_value"]
        from .models import default_base_keys
        ks = default_base_keys(n_layer * len(self.matrix_names))
        self.keys = [{n: ks[l * len(self.matrix_names) + i] for i, n in enumerate(self.matrix_names)}
                     for l in range(n_layer)]

    # ---- one product of the stack: clean, or with every member's rank-r term ----
    def _mm(self, layer: int, name: str, x: torch.Tensor, n: int, T: int, noise: Optional[LmNoise],
            x_relu_square: bool = False) -> torch.Tensor:
        w = self.layers[layer][name]
        tmm = name in TMM_1 or name in TMM_2
        kw = {}
        if noise is not None:
            kw = dict(sigma=noise.sigma, rank=noise.rank, key=self.keys[layer][name], epoch=noise.epoch,
                      first_thread=noise.first_thread, noise_reuse=noise.noise_reuse, tmm=tmm)
            if not tmm and noise.first_thread % 2 == 0 and n % 2 == 0:
                # a member owns T rows and its rank-r factors a few thousand values: generated once per call
                # into a factor cache (the bits the kernels would regenerate tile by tile)
                a, k = w.shape
                kw["cache"] = ops.FactorCache(self.keys[layer][name], noise.epoch, noise.noise_reuse, noise.rank, a, k,
                                              n // 2, first_pair=noise.first_thread // 2, device=self.device)
        return ops.perturbed_linear(x, w, n_pop=n, bm=T, perturb=noise is not None, precision=ops.PRECISION_BF16,
                                    x_relu_square=x_relu_square, **kw)

    def forward_hidden(self, ids: torch.Tensor, noise: Optional[LmNoise] = None) -> torch.Tensor:
        """ids (n, T) int32 -> the (n*T, C) activations after ln_out."""
        n, T = ids.shape
        C, H, S = self.C, self.H, self.S
        rows = n * T
        x = ops.embedding(ids.reshape(rows).contiguous(), self.emb)
        x = ops.layer_norm(x, *self.ln0)
        ns = torch.zeros(rows, dtype=torch.uint8, device=self.device)
        ns[::T] = 1                                                   # every member's first token
        zero_c = torch.zeros(C, device=self.device)
        v_first = None
        for l, w in enumerate(self.layers):
            mm = lambda name, z: self._mm(l, name, z.contiguous(), n, T, noise)
            # ---- TimeMixing, llm.rs:348-479 ----
            xa_ = ops.layer_norm(x, *w["ln1"])
            xr, xw, xk, xv, xa, xg = ops.token_shift_mix_multi(
                xa_, zero_c, [w[nm] for nm in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g")], ns)
            r = mm("receptance", xr)
            # the products of the block; everything element-wise between them and the recurrence, and after
            # it, runs in two kernels (ops.rwkv_mix_prepare / rwkv_mix_finish) instead of some thirty passes
            w_lin = mm("w2", torch.tanh(mm("w1", xw)))
            k = mm("key", xk)
            v = mm("value", xv)
            v_lin = None if l == 0 else mm("v2", torch.tanh(mm("v1", xv)))
            a_lin = mm("a2", torch.tanh(mm("a1", xa)))
            gate = mm("g2", torch.sigmoid(mm("g1", xg)))
            wdec, v, k, nkk, kka = ops.rwkv_mix_prepare(w_lin, v, v_lin, v_first, a_lin, k, w["w0"],
                                                        None if l == 0 else w["v0"], w["a0"], w["k_k"], w["k_a"], H)
            if l == 0:
                v_first = v
            shp = lambda t_: t_.view(n, T, H, S)
            state = torch.zeros(n, H, S, S, device=self.device)
            out = ops.wkv7(shp(r), shp(wdec), shp(k), shp(v), shp(nkk), shp(kka), state)
            y = ops.group_norm(out.reshape(rows, C), H, *w["ln_x"], eps=64e-5)
            y = ops.rwkv_mix_finish(y, r, k, v, gate, w["r_k"].reshape(-1), H)
            ops.add_inplace(x, mm("output", y))
            del xr, xw, xk, xv, xa, xg, r, k, v, gate, out, y, wdec, state, nkk, kka, w_lin, v_lin, a_lin
            # ---- ChannelMixing, llm.rs:192-213 ----
            xc = ops.layer_norm(x, *w["ln2"])
            # k = relu(key(x))^2 (llm.rs:208) is applied where the value product's prepass reads its input
            kf = mm("ffn_key", ops.token_shift_mix(xc, zero_c, w["ffn_x_k"], ns))
            ops.add_inplace(x, self._mm(l, "ffn_value", kf, n, T, noise, x_relu_square=True))
            del xc, kf
        return ops.layer_norm(x, *self.ln_out)

    def fitness(self, ids: torch.Tensor, noise: Optional[LmNoise] = None, chunk_members: int = 256,
                head_members: int = 64, want_logits: bool = False):
        """Mean next-token log-likelihood per member (ids (n, T) int32).  The population is walked
        in chunks of whole antithetic pairs; inside a chunk the head's logits (rows x padded vocab)
        are produced and scored `head_members` members at a time."""
        n, T = ids.shape
        out = torch.empty(n, dtype=torch.float32, device=self.device)
        chunk_members = max(2, chunk_members - chunk_members % 2)
        kept = []
        for lo in range(0, n, chunk_members):
            hi = min(n, lo + chunk_members)
            nz = None
            if noise is not None:
                nz = LmNoise(noise.sigma, noise.rank, noise.epoch, noise.first_thread + lo, noise.noise_reuse)
            part = ids[lo:hi].contiguous()
            h = self.forward_hidden(part, nz)
            for a0 in range(0, hi - lo, head_members):
                a1 = min(hi - lo, a0 + head_members)
                hx = h[a0 * T:a1 * T]
                logits = ops.perturbed_linear(hx, self.head, n_pop=1, bm=hx.shape[0], perturb=False,
                                              precision=ops.PRECISION_BF16)
                out[lo + a0:lo + a1] = self._score(logits, part[a0:a1], a1 - a0, T)
                if want_logits:
                    kept.append(logits[:, :self.vocab].clone())
                del logits
            del h
        return (out, torch.cat(kept)) if want_logits else out

    def _score(self, logits: torch.Tensor, ids: torch.Tensor, n: int, T: int) -> torch.Tensor:
        # the padded head rows are zero weights: their logits exist in memory but are outside [0, vocab)
        import ctypes as C_
        from . import _lib
        from .core import current_stream, get_context
        scratch = torch.empty(n * T, dtype=torch.float32, device=self.device)
        res = torch.empty(n, dtype=torch.float32, device=self.device)
        ctx = get_context(self.device)
        flat = ids.reshape(-1).contiguous()
        _lib.check(_lib.load().hses_token_fitness(ctx.handle, current_stream(), C_.c_void_p(logits.data_ptr()),
                                                  logits.stride(0), C_.c_void_p(flat.data_ptr()), n, 1, T, self.vocab,
                                                  1.0, C_.c_void_p(scratch.data_ptr()), C_.c_void_p(res.data_ptr())))
        return res
