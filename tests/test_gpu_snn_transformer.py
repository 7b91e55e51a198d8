"""SnnTransformer.forward_batched (hyperscalees-models/src/snn_transformer.rs:345-413) assembled
from the library's kernels against a numpy composition of the CPU restatement's pieces (per-member
do_mm with the seeded factors, rate_encode, continuous attention) on the same seeded inputs."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def oracle_forward(oracle, model, x, noise):
    f32 = np.float32
    P = [p.cpu().numpy() for p in model.params()]
    T, n, _ = x.shape
    nt, tin, d, H, hd = model.num_tokens, model.token_in_dim, model.d_model, model.num_heads, model.head_dim

    def nn(idx, xin, w):
        out = np.empty(xin.shape[:-1] + (w.shape[0],), f32)
        for j in range(xin.shape[0]):
            if noise is None:
                out[j] = oracle.do_mm(xin[j], w, 0.0, 1, 0)
            else:
                out[j] = oracle.do_mm(xin[j], w, noise.sigma, noise.rank, noise.base_keys[idx],
                                      iterinfo=(noise.epoch, noise.first_thread + j))
        return out

    rates = []
    for idx in range(3):
        acc = np.zeros((n, nt, d), f32)
        for t in range(T):
            acc = (acc + nn(idx, x[t].reshape(n, nt, tin), P[idx])).astype(f32)
        rates.append(oracle.rate_encode((acc * f32(1.0 / T)).astype(f32), model.proj_gain))
    xh = ((rates[0] + rates[1] + rates[2]) / f32(3.0)).astype(f32) + P[3][None]
    if noise is not None and noise.pos_emb is not None:
        xh = xh + noise.pos_emb.cpu().numpy()
    beta_raw = np.broadcast_to(P[-1].reshape(1, 1), (n, 1)).astype(f32)
    if noise is not None and noise.beta is not None:
        beta_raw = beta_raw + noise.beta.cpu().numpy()
    beta = np.log1p(np.exp(beta_raw)).astype(f32).reshape(n)
    for b in range(len(model.blocks)):
        base = model.block_base(b)
        blk = model.blocks[b]
        heads = []
        for h in range(H):
            q = nn(base + 3 * h, xh, blk["q"][h].cpu().numpy())
            k = nn(base + 3 * h + 1, xh, blk["k"][h].cpu().numpy())
            v = nn(base + 3 * h + 2, xh, blk["v"][h].cpu().numpy())
            o = np.stack([oracle.spiking_attention(q[j], k[j], v[j], 2, float(beta[j]), model.tau_a, 0.0,
                                                   model.g_inh, model.n_iter)[0] for j in range(n)])
            heads.append(o)
        concat = np.concatenate(heads, axis=2).astype(f32)
        xh = (xh + nn(base + 3 * H, concat, blk["o"].cpu().numpy())).astype(f32)
        ff1 = nn(base + 3 * H + 1, xh, blk["ff1"].cpu().numpy())
        act = (ff1 * (f32(1.0) / (f32(1.0) + np.exp(-ff1)))).astype(f32)
        xh = (xh + nn(base + 3 * H + 2, act, blk["ff2"].cpu().numpy())).astype(f32)
    pooled = xh.mean(axis=1, dtype=f32)
    logits = nn(model.out_param_index(), pooled[:, None, :], P[-3])[:, 0, :]
    gain = np.broadcast_to(P[-2].reshape(1, 1), (n, 1)).astype(f32)
    if noise is not None and noise.out_gain is not None:
        gain = gain + noise.out_gain.cpu().numpy()
    return (logits * gain).astype(f32)


@pytest.mark.parametrize("perturbed", [False, True])
def test_forward_batched_matches_oracle_composition(hs, oracle, perturbed):
    from hyperscalees_b200.snn_transformer import SnnTransformer, TrainNoise
    from hyperscalees_b200.models import default_base_keys
    tin, nt, classes, d, H, blocks, T, n = 8, 5, 3, 32, 2, 2, 3, 6
    model = SnnTransformer(tin, nt, classes, d, H, blocks, device="cuda", seed=4)
    g = np.random.default_rng(9)
    model.pos_emb = torch.as_tensor(g.standard_normal((nt, d)).astype(np.float32) * 0.1, device="cuda")
    x = (g.random((T, n, nt * tin)) < 0.3).astype(np.float32)
    noise = None
    if perturbed:
        keys = default_base_keys(len(model.params()))
        dn = lambda *s: torch.as_tensor(g.standard_normal(s).astype(np.float32) * 0.05, device="cuda")
        noise = TrainNoise(sigma=0.05, rank=4, base_keys=keys, epoch=2, first_thread=4,
                           pos_emb=dn(n, nt, d), out_gain=dn(n, 1), beta=dn(n, 1))
    got = model.forward_batched(torch.as_tensor(x, device="cuda"), noise).cpu().numpy()
    want = oracle_forward(oracle, model, x, noise)
    assert got.shape == (n, classes)
    assert np.abs(got - want).max() <= 1e-4 * max(1.0, np.abs(want).max())
    if perturbed:
        # factors generated once for the chunk give the bits of regenerated ones
        noise.caches = model.build_caches(noise, n)
        cached = model.forward_batched(torch.as_tensor(x, device="cuda"), noise).cpu().numpy()
        assert np.array_equal(cached, got)
        # antithetic partners (thread ids 4 and 5) see different weights: their logits differ
        clean = model.forward_batched(torch.as_tensor(x, device="cuda"), None).cpu().numpy()
        assert np.abs(got - clean).max() > 1e-4


def test_params_and_es_map_layout():
    """snn_transformer.rs:204-253: parameter order and es classes."""
    from hyperscalees_b200.snn_transformer import SnnTransformer
    from hyperscalees_b200.noiser import MM_PARAM, EMB_PARAM, PARAM
    m = SnnTransformer(4, 3, 2, 8, 2, 2, device="cuda")
    ps, es = m.params(), m.es_map()
    assert len(ps) == len(es) == 3 + 1 + 2 * (3 * 2 + 3) + 1 + 2
    assert es[3] == EMB_PARAM and es[-1] == PARAM and es[-2] == PARAM and es.count(MM_PARAM) == len(es) - 3
    assert m.block_base(1) == 4 + 9 and m.out_param_index() == 4 + 18
    assert tuple(ps[4].shape) == (4, 8) and tuple(ps[m.out_param_index()].shape) == (2, 8)
    with pytest.raises(ValueError):
        m.forward_batched(torch.zeros(2, 3, 11, device="cuda"))
