"""RWKV-7 state recurrence and the spiking self-attention core against the CPU oracle."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.as_tensor(np.ascontiguousarray(a), device="cuda")


def test_wkv7_reference_decay_case(hs):
    # hyperscalees-models/src/llm.rs:1040-1095: k = v = a = b = 0, decay 0.5 per step
    from hyperscalees_b200 import ops
    S = 32  # the reference case is 2x2; embed it in the top-left corner of a 32x32 head
    st = torch.zeros(1, 2, S, S, device="cuda")
    st[0, 0, :2, :2] = torch.tensor([[1.0, 2.0], [3.0, 4.0]])
    st[0, 1, :2, :2] = torch.tensor([[5.0, 6.0], [7.0, 8.0]])
    r = torch.zeros(1, 2, 2, S, device="cuda")
    r[0, 0, 0, 0] = 1.0; r[0, 0, 1, 1] = 1.0; r[0, 1, :, :2] = 1.0
    z = torch.zeros_like(r)
    w = torch.full_like(r, math.log(math.log(2.0)))
    out = ops.wkv7(r, w, z, z, z, z, st)
    assert torch.allclose(out[0, 0, 0, :2].cpu(), torch.tensor([0.5, 1.5]), atol=1e-5)
    assert torch.allclose(out[0, 0, 1, :2].cpu(), torch.tensor([3.0, 4.0]), atol=1e-5)
    assert torch.allclose(out[0, 1, 0, :2].cpu(), torch.tensor([0.75, 1.75]), atol=1e-5)
    assert torch.allclose(out[0, 1, 1, :2].cpu(), torch.tensor([2.75, 3.75]), atol=1e-5)
    assert torch.allclose(st[0, 0, :2, :2].cpu(), torch.tensor([[0.25, 0.5], [0.75, 1.0]]), atol=1e-5)
    assert torch.allclose(st[0, 1, :2, :2].cpu(), torch.tensor([[1.25, 1.5], [1.75, 2.0]]), atol=1e-5)


@pytest.mark.parametrize("n_seq,T,H,S", [(1, 5, 2, 64), (3, 16, 12, 64), (2, 7, 3, 32)])
def test_wkv7_matches_oracle(hs, oracle, n_seq, T, H, S):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(T * 10 + H)
    mk = lambda s: (g.standard_normal((n_seq, T, H, S)) * s).astype(np.float32)
    r, k, v, a, b = mk(1.0), mk(0.3), mk(1.0), mk(0.1), mk(0.1)
    w = (g.standard_normal((n_seq, T, H, S)) * 0.5 - 1.0).astype(np.float32)
    st0 = (g.standard_normal((n_seq, H, S, S)) * 0.1).astype(np.float32)
    ns = np.zeros((n_seq, T), np.uint8)
    ns[0, T // 2] = 1
    st = dev(st0).clone()
    out = ops.wkv7(dev(r), dev(w), dev(k), dev(v), dev(a), dev(b), st, dev(ns)).cpu().numpy()
    for s in range(n_seq):
        want_st, want = oracle.wkv7(r[s], w[s], k[s], v[s], a[s], b[s], st0[s], ns[s])
        scale = max(1.0, np.abs(want).max())
        assert np.abs(out[s] - want).max() <= 1e-5 * scale
        assert np.abs(st[s].cpu().numpy() - want_st).max() <= 1e-5 * max(1.0, np.abs(want_st).max())


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("n_seq,tokens,heads,hd", [(2, 64, 4, 16), (3, 16, 1, 8), (1, 50, 2, 64), (2, 50, 2, 32),
                                                   (1, 7, 3, 16), (1, 128, 1, 32), (1, 128, 2, 64), (1, 100, 1, 64)])
def test_spiking_attention_matches_oracle(hs, oracle, mode, n_seq, tokens, heads, hd):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(tokens + hd)
    # firing rates of T = 4 LIF steps: multiples of 1/4
    mk = lambda: (g.integers(0, 5, (n_seq, tokens, heads * hd)) / 4.0).astype(np.float32)
    Q, K, V = mk(), mk(), mk()
    O, A = ops.spiking_attention(dev(Q), dev(K), dev(V), heads, mode=mode, beta=1.0 / math.sqrt(hd), tau_m=2.0,
                                 v_th=0.3, g_inh=0.5, n_iter=8, want_weights=True)
    O, A = O.cpu().numpy(), A.cpu().numpy()
    for s in range(n_seq):
        for h in range(heads):
            sl = slice(h * hd, (h + 1) * hd)
            wo, wa = oracle.spiking_attention(Q[s][:, sl], K[s][:, sl], V[s][:, sl], mode, 1.0 / math.sqrt(hd),
                                              2.0, 0.3, 0.5, 8)
            assert np.array_equal(A[s, h], wa) or np.abs(A[s, h] - wa).max() <= 1e-6
            assert np.abs(O[s][:, sl] - wo).max() <= 1e-5 * max(1.0, np.abs(wo).max())
            if mode == 0:
                # rates that are multiples of 1/4: every score is exact, with or without fused multiply-adds
                assert np.array_equal(A[s, h], wa)
    if mode == 1:
        rows = A.sum(-1)
        assert ((np.abs(rows - 1.0) < 1e-4) | (rows == 0.0)).all()  # a row sums to one whenever any key fired


def test_layer_and_group_norm_match_oracle():
    """llm.rs:930-999 (hand-computed cases, via the oracle's pins) and random shapes."""
    from hyperscalees_b200 import ops
    from oracle import oracle
    g = np.random.default_rng(3)
    x = np.array([[1, 2, 3, 4], [10, 20, 30, 40]], dtype=np.float32)
    w, b = np.array([2.0, 1.0, 0.5, 1.0], np.float32), np.array([1.0, 0.0, 0.5, -1.0], np.float32)
    got = ops.layer_norm(dev(x), dev(w), dev(b)).cpu().numpy()
    assert np.abs(got - np.array([[-1.6832, -0.4472, 0.7236, 0.3416]] * 2)).max() <= 1e-4
    x = g.standard_normal((37, 768)).astype(np.float32) * 3 + 1
    w, b = g.standard_normal(768).astype(np.float32), g.standard_normal(768).astype(np.float32)
    assert np.allclose(ops.layer_norm(dev(x), dev(w), dev(b)).cpu().numpy(), oracle.layer_norm(x, w, b), rtol=1e-4, atol=1e-4)
    # group norm: rank 3 (hand case) and the rank-2 form TimeMixing uses (groups = heads)
    x3 = np.arange(1, 17, dtype=np.float32).reshape(2, 4, 2)
    got = ops.group_norm(dev(x3), 2, dev(np.ones(4, np.float32)), dev(np.zeros(4, np.float32))).cpu().numpy()
    assert np.abs(got.reshape(-1) - np.tile([-1.34164, -0.44721, 0.44721, 1.34164], 4)).max() <= 1e-4
    x2 = g.standard_normal((50, 768)).astype(np.float32)
    assert np.allclose(ops.group_norm(dev(x2), 12, dev(w), dev(b), eps=64e-5).cpu().numpy(),
                       oracle.group_norm(x2, 12, w, b, eps=64e-5), rtol=1e-4, atol=1e-4)
    x3 = g.standard_normal((5, 24, 7)).astype(np.float32)
    w3, b3 = g.standard_normal(24).astype(np.float32), g.standard_normal(24).astype(np.float32)
    assert np.allclose(ops.group_norm(dev(x3), 4, dev(w3), dev(b3)).cpu().numpy(), oracle.group_norm(x3, 4, w3, b3),
                       rtol=1e-4, atol=1e-4)


def test_channel_mixing_matches_oracle_and_reference_case():
    """llm.rs:1003-1036 (T = 2, C = 1 hand case) and a random block with sequence restarts."""
    from hyperscalees_b200 import models, ops
    from oracle import oracle
    cm = models.ChannelMixing(dev(np.array([2.0], np.float32)), dev(np.array([[1.0]], np.float32)),
                              dev(np.array([[1.0]], np.float32)))
    out, st = cm.forward(dev(np.array([[3.0], [5.0]], np.float32)), dev(np.array([[1.0]], np.float32)), 2,
                         torch.tensor([0, 0]))
    assert np.abs(out.cpu().numpy().reshape(-1) - np.array([0.0, 1.0])).max() <= 1e-4
    assert abs(st.cpu().numpy().reshape(-1)[0] - 5.0) <= 1e-4
    g = np.random.default_rng(8)
    T, c, f = 33, 64, 256
    x = g.standard_normal((T, c)).astype(np.float32)
    state = g.standard_normal(c).astype(np.float32)
    x_k = g.random(c).astype(np.float32)
    wk = (g.standard_normal((f, c)) / np.sqrt(c)).astype(np.float32)
    wv = (g.standard_normal((c, f)) / np.sqrt(f)).astype(np.float32)
    ns = np.zeros(T, np.uint8); ns[[0, 9, 20]] = 1
    cm = models.ChannelMixing(dev(x_k), dev(wk), dev(wv))
    out, st = cm.forward(dev(x), dev(state), 30, torch.from_numpy(ns))
    want, wst = oracle.channel_mix(x, state, x_k, wk, wv, 30, ns)
    assert np.abs(out.cpu().numpy() - want).max() <= 1e-4 * max(np.abs(want).max(), 1.0)
    assert np.array_equal(st.cpu().numpy().reshape(-1), wst)
    # the token shift alone is exact
    assert np.array_equal(ops.token_shift_mix(dev(x), dev(state), dev(x_k), torch.from_numpy(ns)).cpu().numpy(),
                          oracle.token_shift_mix(x, state, x_k, ns))


@pytest.mark.parametrize("n_seq,tokens,heads,hd", [(3, 17, 4, 16), (1, 128, 1, 64)])
def test_continuous_hopfield_attention_and_rate_encode(hs, oracle, n_seq, tokens, heads, hd):
    """snn_transformer.rs:80-116: continuous rates, Hopfield relaxation, softmax rows that sum to one
    (the reference asserts the row sums in snn_attention.rs:374-399).  The second shape is the
    largest the entry point takes (its rows do not fit the register kernel's shared memory)."""
    from hyperscalees_b200 import ops
    g = np.random.default_rng(21)
    p = g.standard_normal((n_seq, tokens, heads * hd)).astype(np.float32) * 2
    rates = ops.rate_encode(dev(p), 4.0).cpu().numpy()
    assert np.abs(rates - oracle.rate_encode(p, 4.0)).max() <= 1e-6
    assert (rates > 0).all() and (rates < 1).all()
    Q, K, V = rates, np.roll(rates, 1, axis=1).copy(), np.roll(rates, 2, axis=2).copy()
    O, A = ops.spiking_attention(dev(Q), dev(K), dev(V), heads, mode=2, beta=2.0, tau_m=2.0, v_th=0.0, g_inh=0.5,
                                 n_iter=8, want_weights=True)
    O, A = O.cpu().numpy(), A.cpu().numpy()
    assert np.abs(A.sum(-1) - 1.0).max() <= 1e-4
    for s in range(n_seq):
        for h in range(heads):
            sl = slice(h * hd, (h + 1) * hd)
            wo, wa = oracle.spiking_attention(Q[s][:, sl], K[s][:, sl], V[s][:, sl], 2, 2.0, 2.0, 0.0, 0.5, 8)
            assert np.abs(A[s, h] - wa).max() <= 2e-6
            assert np.abs(O[s][:, sl] - wo).max() <= 1e-5
