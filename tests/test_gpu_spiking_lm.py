"""The token-level spiking transformer against the numpy composition of the CPU restatement's
pieces (oracle/spiking_lm.py), member by member, plus its building blocks alone."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.as_tensor(np.ascontiguousarray(a), device="cuda")


def test_embedding_gather_with_rank_r_term(hs, oracle):
    from hyperscalees_b200 import ops
    from oracle import spiking_lm as SL
    g = np.random.default_rng(0)
    vocab, d, L, rank, n, seqs, sigma, key = 50, 32, 10, 4, 6, 2, 0.3, 0x9E3779B97F4A7C15
    table = g.standard_normal((vocab, d)).astype(np.float32)
    pos = g.standard_normal((L, d)).astype(np.float32)
    ids = g.integers(0, vocab, (n, seqs, L)).astype(np.int32)
    A, B = ops.lora_factors(key, 0, 0, rank, vocab, d, ops.base_sigma(sigma, rank), n, first_thread=4)
    got = ops.embedding(dev(ids.reshape(-1)), dev(table), dev(pos), A, B, rows_per_member=seqs * L).cpu().numpy()
    for m in range(n):
        want = SL.embed(ids[m].reshape(-1), table, pos, sigma, rank, key, (0, 4 + m))
        assert np.array_equal(got[m * seqs * L:(m + 1) * seqs * L], want)
    clean = ops.embedding(dev(ids.reshape(-1)), dev(table)).cpu().numpy()
    assert np.array_equal(clean, table[ids.reshape(-1)])
    # an id outside the table is reported through the device status word
    from hyperscalees_b200 import core
    bad = ids.reshape(-1).copy()
    bad[3] = vocab
    ops.embedding(dev(bad), dev(table))
    assert core.get_context(0).device_status() & (1 << 15)


def test_lif_rate_swish_and_add(hs, oracle):
    from hyperscalees_b200 import ops
    from oracle import spiking_lm as SL
    g = np.random.default_rng(1)
    cur = (g.standard_normal((37, 19)) * 0.8).astype(np.float32)
    for T, tau, vth in ((4, 2.0, 0.3), (8, 20.0, 0.05), (1, 1.0, 0.5)):
        got = ops.lif_rate(dev(cur), T, tau, vth).cpu().numpy()
        assert np.array_equal(got, SL.lif_rate(cur, T, tau, vth))
    x = (g.standard_normal(1003) * 3).astype(np.float32)
    assert np.abs(ops.swish(dev(x)).cpu().numpy() - SL.swish(x)).max() <= 1e-6
    a, b = g.standard_normal(1003).astype(np.float32), g.standard_normal(1003).astype(np.float32)
    assert np.array_equal(ops.add_inplace(dev(a), dev(b)).cpu().numpy(), a + b)


def test_causal_spike_product_attention(hs, oracle):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(2)
    for n_seq, tokens, heads, hd in ((2, 64, 4, 16), (1, 10, 2, 16), (1, 33, 1, 32), (1, 50, 1, 64), (2, 9, 3, 8)):
        mk = lambda: (g.integers(0, 5, (n_seq, tokens, heads * hd)) / 4.0).astype(np.float32)
        Q, K, V = mk(), mk(), mk()
        for want_w in (False, True):
            res = ops.spiking_attention(dev(Q), dev(K), dev(V), heads, mode=3, beta=0.25, want_weights=want_w)
            O_, A_ = (res if want_w else (res, None))
            O_ = O_.cpu().numpy()
            for s in range(n_seq):
                for h in range(heads):
                    sl = slice(h * hd, (h + 1) * hd)
                    wo, wa = oracle.spiking_attention(Q[s][:, sl], K[s][:, sl], V[s][:, sl], 3, 0.25)
                    assert np.abs(O_[s][:, sl] - wo).max() <= 1e-5 * max(1.0, np.abs(wo).max())
                    assert np.allclose(np.triu(wa, 1), 0.0)
                    if want_w:
                        assert np.array_equal(A_[s, h].cpu().numpy(), wa)


def _np_model(m):
    return {"emb": m.emb.cpu().numpy(), "pos_emb": m.pos_emb.cpu().numpy(), "out": m.out.cpu().numpy(),
            "blocks": [{k: ([w.cpu().numpy() for w in v] if isinstance(v, list) else v.cpu().numpy())
                        for k, v in blk.items()} for blk in m.blocks],
            "T": m.T, "tau_m": m.tau_m, "v_th": m.v_th, "beta": m.beta, "num_heads": m.num_heads}


@pytest.mark.parametrize("perturb", [False, True])
def test_forward_and_fitness_match_the_cpu_composition(hs, oracle, perturb):
    from hyperscalees_b200 import models, ops
    from hyperscalees_b200.spiking_lm import LmNoise, SpikingLM
    from oracle import spiking_lm as SL
    vocab, L, d, H, blocks, rank, sigma, n, seqs = 48, 12, 32, 2, 2, 4, 0.05, 6, 2
    m = SpikingLM(vocab, L, d, H, blocks, mlp_ratio=4, T=4, seed=2)
    g = np.random.default_rng(2)
    ids = g.integers(0, vocab, (n, seqs, L)).astype(np.int32)
    keys = models.default_base_keys(len(m.params()))
    noise = LmNoise(sigma, rank, keys, epoch=0, first_thread=2) if perturb else None
    logits = m.forward_population(dev(ids), noise).cpu().numpy().reshape(n, seqs * L, vocab)
    fit = m.fitness(dev(ids), noise, chunk_members=4).cpu().numpy()
    npm = _np_model(m)
    for j in range(n):
        info = (0, 2 + j) if perturb else None
        want = SL.member_forward(npm, ids[j], sigma, rank, keys, info)
        assert np.abs(logits[j] - want).max() <= 2e-4 * max(1.0, np.abs(want).max())
        wf = SL.member_fitness(want, ids[j])
        assert abs(fit[j] - wf) <= 2e-4 * max(1.0, abs(wf))
    if perturb:
        # antithetic partners differ, and the perturbation reaches the logits
        assert np.abs(logits[0] - logits[1]).max() > 0
