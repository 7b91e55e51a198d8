"""CPU restatement of the RWKV-7 language-model forward for ONE member, composed from the restated
pieces of oracle.py (token shift, WKV-7 recurrence, norms, factors).  Test infrastructure: only
tests/ import it.

Follows src/hyperscalees/models/llm/rwkv7.py:222-253 (`forward_seq`: ln0, then per block
ln1 -> TimeMixing -> residual, ln2 -> ChannelMixing -> residual) and llm/llm.py:91-104 (embed,
forward_seq, ln_out + head), with the block algebra of hyperscalees-models/src/llm.rs:348-479 and
192-213.  Products round their operands to bf16 and accumulate wide (the model's weights are bf16
values); the member's low-rank term is fp32: do_mm (eggroll.rs:419-446) for Linear weights,
do_Tmm (eggroll.rs:450-477) for the (in, out) TMM weights.  Parity unpinned beyond the pieces: the
reference has no output for this composition that could be produced here.
"""
from __future__ import annotations

import numpy as np

from . import oracle as O

f32 = np.float32


def bf16r(x):
    """round-to-nearest-even to bf16, returned as float32"""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(x))


def layer_norm(x, wb):
    return O.layer_norm(x, wb[0], wb[1])


def product(x, w_out_in, noise, key, tmm, rows_in_call=None):
    """x (T, in), weight held (out, in).  noise = (sigma, rank, epoch, thread_id, noise_reuse) or None.
    The operands are rounded to bf16 where the library's bf16 product exists (its tensor-core
    kernel: output width a multiple of 32, input width a multiple of 8, the call's rows a multiple
    of 128); anything else is an fp32 product."""
    out_dim, in_dim = w_out_in.shape
    rows = x.shape[0] if rows_in_call is None else rows_in_call
    if out_dim % 32 == 0 and in_dim % 8 == 0 and rows % 128 == 0:
        base = (bf16r(x).astype(np.float64) @ bf16r(w_out_in).astype(np.float64).T)
    else:
        base = x.astype(np.float64) @ w_out_in.astype(np.float64).T
    if noise is None:
        return base.astype(f32)
    sigma, rank, ep, tid, reuse = noise
    bs = float(f32(sigma) / np.sqrt(f32(rank)))
    if tmm:   # reference parameter (in, out): A (in, r) scaled, B (out, r)
        A, B = O.lora_params(bs, key, rank, ep, tid, in_dim, out_dim, reuse)
        u = (x.astype(np.float64) @ A.astype(np.float64)) @ B.astype(np.float64).T
    else:     # parameter (out, in): A (out, r) scaled, B (in, r)
        A, B = O.lora_params(bs, key, rank, ep, tid, out_dim, in_dim, reuse)
        u = (x.astype(np.float64) @ B.astype(np.float64)) @ A.astype(np.float64).T
    return (base + u).astype(f32)


def member_hidden(model, ids, noise=None, rows_in_call=None):
    """model: dict with emb, ln0, ln_out, layers (list of dicts of numpy arrays as RwkvLM holds them),
    keys (list of dicts), H, S.  ids (T,) -> (T, C) after ln_out."""
    H, S = model["H"], model["S"]
    x = model["emb"][ids].astype(f32)
    T, C = x.shape
    x = layer_norm(x, model["ln0"])
    ns = np.zeros(T, bool)
    ns[0] = True
    zero = np.zeros(C, f32)
    sig = lambda z: (f32(1.0) / (f32(1.0) + np.exp(-z.astype(f32)))).astype(f32)
    v_first = None
    for l, w in enumerate(model["layers"]):
        keys = model["keys"][l]
        mm = lambda name, z: product(z.astype(f32), w[name], noise, keys[name],
                                     len(name) == 2 and name[0] in "wvag" and name[1] in "12", rows_in_call)
        xa_ = layer_norm(x, w["ln1"])
        mix = lambda n: O.token_shift_mix(xa_, zero, w[n], ns)
        xr, xw, xk, xv, xa, xg = (mix(n) for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g"))
        r = mm("receptance", xr)
        inner_w = (w["w0"][None] + mm("w2", np.tanh(mm("w1", xw)))).astype(f32)
        wdec = (-np.logaddexp(f32(0.0), -inner_w) - f32(0.5)).astype(f32)
        k = mm("key", xk)
        v = mm("value", xv)
        if l == 0:
            v_first = v.copy()
        else:
            v = (v + (v_first - v) * sig(w["v0"][None] + mm("v2", np.tanh(mm("v1", xv))))).astype(f32)
        a = sig(w["a0"][None] + mm("a2", np.tanh(mm("a1", xa))))
        gate = mm("g2", sig(mm("g1", xg)))
        kk3 = (k * w["k_k"][None]).reshape(T, H, S)
        kk = (kk3 / np.maximum(np.sqrt((kk3 ** 2).sum(axis=2, keepdims=True)), 1e-12)).reshape(T, C).astype(f32)
        k = (k * (w["k_a"][None] * (a - f32(1.0)) + f32(1.0))).astype(f32)
        sh = lambda z: np.ascontiguousarray(z.reshape(T, H, S).astype(f32))
        _, out = O.wkv7(sh(r), sh(wdec), sh(k), sh(v), sh(-kk), sh(kk * a), np.zeros((H, S, S), f32),
                        ns.astype(np.uint8))
        y = O.group_norm(out.reshape(T, C), H, w["ln_x"][0], w["ln_x"][1], eps=64e-5)
        bonus = (r.reshape(T, H, S) * k.reshape(T, H, S) * w["r_k"].reshape(1, H, S)).sum(axis=2, keepdims=True)
        y = ((y + (bonus * v.reshape(T, H, S)).reshape(T, C)) * gate).astype(f32)
        x = (x + mm("output", y)).astype(f32)
        xc = layer_norm(x, w["ln2"])
        kf = mm("ffn_key", O.token_shift_mix(xc, zero, w["ffn_x_k"], ns))
        kf = (np.maximum(kf, f32(0.0)) ** 2).astype(f32)
        x = (x + mm("ffn_value", kf)).astype(f32)
    return layer_norm(x, model["ln_out"])


def member_fitness(model, ids, noise=None, rows_in_call=None, head_rows_in_call=None):
    """mean over positions 0..T-2 of log_softmax(head(h[t]))[ids[t+1]] (llm.py:91-104 + the trainer's
    token log-likelihood), head product in bf16 like the rest"""
    h = member_hidden(model, ids, noise, rows_in_call)
    logits = product(h, model["head_padded"], None, 0, False, head_rows_in_call)[:, :model["head"].shape[0]]
    lp = O.fitness(logits[:-1], ids[1:].astype(np.int32))
    return f32(lp.astype(np.float64).mean()), logits
