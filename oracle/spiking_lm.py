"""CPU restatement of the token-level spiking transformer's forward pass for one member, composed
from the restated pieces of oracle.py (factors, do_mm, lif_step, the attention core, the
log-softmax fitness).  Test infrastructure: only tests/ import it.

There is no reference output for this composition: the reference holds the block structure
(hyperscalees-models/src/snn_transformer.rs:345-413), the LIF-coded Q/K/V
(src/hyperscalees/models/snn_self_attention.py:114-131) and an unimplemented embedding hook
(src/hyperscalees/noiser/eggroll.py:93).  Parity unpinned beyond those pieces.
"""
from __future__ import annotations

import numpy as np

from . import oracle as O


def base_sigma(sigma: float, rank: int) -> np.float32:
    return np.float32(sigma) / np.sqrt(np.float32(rank))


def embed(ids, table, pos, sigma, rank, key, iterinfo, noise_reuse=0):
    """table[ids] + A[ids] B^T + pos (do_emb: clean gather plus the member's rank-r term); the
    rank-r dot product is summed in index order with every product and sum rounded."""
    x = table[ids].astype(np.float32).copy()
    if iterinfo is not None:
        ep, tid = iterinfo
        A, B = O.lora_params(float(base_sigma(sigma, rank)), key, rank, ep, tid, table.shape[0], table.shape[1],
                             noise_reuse)
        u = np.zeros_like(x)
        for q in range(rank):
            u = (u + (A[ids, q][:, None] * B[None, :, q]).astype(np.float32)).astype(np.float32)
        x = (x + u).astype(np.float32)
    L = pos.shape[0]
    return (x + pos[np.arange(len(ids)) % L]).astype(np.float32)


def lif_rate(cur, T, tau_m, v_th):
    """T steps of lif_step (snn.rs:53-65) on a constant current from v = 0; spikes / T."""
    flat = np.ascontiguousarray(cur, dtype=np.float32).reshape(1, -1)
    rep = np.repeat(flat[None], T, axis=0)                     # (T, 1, n)
    spikes, _ = O.run_lif(rep, np.zeros_like(flat), tau_m, v_th)
    s = np.zeros(flat.shape[1], np.float32)
    for t in range(T):
        s = (s + spikes[t, 0]).astype(np.float32)
    return (s / np.float32(T)).astype(np.float32).reshape(cur.shape)


def swish(x):
    x = x.astype(np.float32)
    return (x * (np.float32(1.0) / (np.float32(1.0) + np.exp(-x, dtype=np.float32)))).astype(np.float32)


def member_forward(model, ids, sigma, rank, keys, iterinfo, noise_reuse=0, acc64=False):
    """model: dict of numpy parameters (emb, pos_emb, blocks [{q: [...], k: [...], v: [...], o, ff1,
    ff2}], out) and scalars (T, tau_m, v_th, beta, num_heads); ids (seqs, L).  Returns logits
    (seqs*L, vocab) before the output gain."""
    seqs, L = ids.shape
    H = model["num_heads"]
    d = model["emb"].shape[1]
    hd = d // H
    mm = lambda idx, w, x: O.do_mm(x, w, sigma, rank, keys[idx], iterinfo, noise_reuse, acc64)
    x = embed(ids.reshape(-1), model["emb"], model["pos_emb"], sigma, rank, keys[0], iterinfo, noise_reuse)
    idx = 2
    for blk in model["blocks"]:
        Q, K, V = (np.empty((seqs * L, d), np.float32) for _ in range(3))
        for h in range(H):
            sl = slice(h * hd, (h + 1) * hd)
            Q[:, sl] = lif_rate(mm(idx + 3 * h, blk["q"][h], x), model["T"], model["tau_m"], model["v_th"])
            K[:, sl] = lif_rate(mm(idx + 3 * h + 1, blk["k"][h], x), model["T"], model["tau_m"], model["v_th"])
            V[:, sl] = lif_rate(mm(idx + 3 * h + 2, blk["v"][h], x), model["T"], model["tau_m"], model["v_th"])
        attn = np.empty_like(Q)
        for s in range(seqs):
            rows = slice(s * L, (s + 1) * L)
            for h in range(H):
                sl = slice(h * hd, (h + 1) * hd)
                attn[rows, sl], _ = O.spiking_attention(Q[rows, sl], K[rows, sl], V[rows, sl], 3, model["beta"])
        x = (x + mm(idx + 3 * H, blk["o"], attn)).astype(np.float32)
        act = swish(mm(idx + 3 * H + 1, blk["ff1"], x))
        x = (x + mm(idx + 3 * H + 2, blk["ff2"], act)).astype(np.float32)
        idx += 3 * H + 3
    return mm(idx, model["out"], x)


def member_fitness(logits, ids, gain=1.0):
    """mean over sequences and positions 0..L-2 of log_softmax(gain * logits[s, t])[ids[s, t+1]]"""
    seqs, L = ids.shape
    lg = (logits.astype(np.float32) * np.float32(gain)).reshape(seqs, L, -1)
    tot = np.float64(0.0)
    for s in range(seqs):
        lp = O.fitness(lg[s, :L - 1], ids[s, 1:].astype(np.int32))
        tot += np.float64(lp.astype(np.float64).sum())
    return np.float32(tot / (seqs * (L - 1)))
