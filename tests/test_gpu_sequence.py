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
@pytest.mark.parametrize("n_seq,tokens,heads,hd", [(2, 64, 4, 16), (3, 16, 1, 8), (1, 50, 2, 64)])
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
    if mode == 1:
        rows = A.sum(-1)
        assert ((np.abs(rows - 1.0) < 1e-4) | (rows == 0.0)).all()  # a row sums to one whenever any key fired
