"""Parity of the perturbed linear layer (+ fused LIF step) with the CPU oracle.

Matmul accumulation order is not pinned by the reference (third-party GEMM),
so potentials are compared with a tolerance and spikes with the mismatch
criterion: at most 1e-4 of the spikes may differ, and only where the
double-accumulated membrane potential lies within 1e-5 of the threshold."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

KEY = 0x3C6EF372FE94F82A


def dev(a):
    return torch.as_tensor(np.ascontiguousarray(a), device="cuda")


def oracle_mm(oracle, x, w, sigma, rank, key, epoch, first, reuse, acc64=False):
    n_pop = x.shape[-3]
    flat = x.reshape(-1, n_pop, x.shape[-2], x.shape[-1])
    out = np.empty(flat.shape[:3] + (w.shape[0],), np.float32)
    for t in range(flat.shape[0]):
        for i in range(n_pop):
            out[t, i] = oracle.do_mm(flat[t, i], w, sigma, rank, key, (epoch, first + i), reuse, acc64)
    return out.reshape(-1, w.shape[0])


@pytest.mark.parametrize("algo", [1])
@pytest.mark.parametrize("n_pop,bm,k,a,rank,t_steps,first", [
    (4, 16, 64, 48, 4, 1, 0),
    (5, 3, 37, 19, 2, 1, 1),      # ragged sizes, odd first member
    (6, 2, 128, 130, 16, 3, 2),   # several time steps share a member's noise
    (2, 64, 784, 128, 4, 1, 0),   # SNN first-layer shape
    (3, 1, 16, 8, 1, 1, 4),
])
def test_do_mm_population_matches_oracle(hs, oracle, algo, n_pop, bm, k, a, rank, t_steps, first):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(n_pop * 100 + k)
    x = g.standard_normal((t_steps, n_pop, bm, k)).astype(np.float32)
    w = (g.standard_normal((a, k)) / np.sqrt(k)).astype(np.float32)
    sigma = 0.5
    got = ops.perturbed_linear(dev(x), dev(w), n_pop=n_pop, bm=bm, t_steps=t_steps, sigma=sigma,
                               rank=rank, key=KEY, epoch=3, first_thread=first, noise_reuse=1,
                               algo=algo).cpu().numpy()
    want = oracle_mm(oracle, x, w, sigma, rank, KEY, 3, first, 1, acc64=True)
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 2e-5 * max(scale, 1.0)
    # the perturbation is really there: the clean product differs
    clean = ops.perturbed_linear(dev(x), dev(w), n_pop=n_pop, bm=bm, t_steps=t_steps, perturb=False,
                                 algo=algo).cpu().numpy()
    assert np.abs(clean - x.reshape(-1, k) @ w.T).max() <= 2e-5 * max(scale, 1.0)
    assert np.abs(clean - got).max() > 1e-3


@pytest.mark.parametrize("algo", [1])
def test_pitched_operands(hs, oracle, algo):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(0)
    n_pop, bm, k, a = 3, 4, 100, 60
    xb = torch.zeros(n_pop * bm, 128, device="cuda")
    wb = torch.zeros(a, 104, device="cuda")
    ob = torch.full((n_pop * bm, 64), float("nan"), device="cuda")
    x = g.standard_normal((n_pop, bm, k)).astype(np.float32)
    w = g.standard_normal((a, k)).astype(np.float32)
    xb[:, :k] = dev(x.reshape(-1, k))
    wb[:, :k] = dev(w)
    ops.perturbed_linear(xb[:, :k], wb[:, :k], n_pop=n_pop, bm=bm, sigma=0.1, rank=4, key=KEY,
                         out=ob[:, :a], algo=algo)
    want = oracle_mm(oracle, x, w, 0.1, 4, KEY, 0, 0, 0, acc64=True)
    assert np.abs(ob[:, :a].cpu().numpy() - want).max() <= 2e-5 * np.abs(want).max()
    assert torch.isnan(ob[:, a:]).all()  # the padding columns were not touched


@pytest.mark.parametrize("algo", [1])
@pytest.mark.parametrize("tau_m,v_th", [(20.0, 0.3), (2.0, 1.0)])
def test_fused_lif_spikes(hs, oracle, algo, tau_m, v_th):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(7)
    n_pop, bm, k, a, rank = 32, 16, 256, 256, 16
    x = g.standard_normal((n_pop, bm, k)).astype(np.float32)
    w = g.standard_normal((a, k)).astype(np.float32)
    sigma = 0.02
    got_s, got_c = ops.perturbed_linear(dev(x), dev(w), n_pop=n_pop, bm=bm, sigma=sigma, rank=rank,
                                        key=KEY, lif=True, tau_m=tau_m, v_th=v_th,
                                        want_potentials=True, algo=algo)
    want_s = oracle.perturbed_linear_lif(x, w, sigma, rank, KEY, tau_m=tau_m, v_th=v_th)
    _, c64 = oracle.perturbed_linear_lif(x, w, sigma, rank, KEY, tau_m=tau_m, v_th=v_th, acc64=True,
                                         want_potentials=True)
    got_s = got_s.cpu().numpy().reshape(want_s.shape)
    got_c = got_c.cpu().numpy().reshape(c64.shape)
    assert set(np.unique(got_s)) <= {0.0, 1.0}
    assert np.abs(got_c - c64).max() <= 1e-5 * max(1.0, np.abs(c64).max())
    mism = got_s != want_s
    assert mism.mean() <= 1e-4
    assert (np.abs(c64[mism] - v_th) < 1e-5).all()
    assert 0.05 < got_s.mean() < 0.95


def test_shape_errors_are_reported(hs):
    from hyperscalees_b200 import ops
    x = torch.zeros(8, 16, device="cuda")
    w = torch.zeros(4, 15, device="cuda")
    with pytest.raises(ValueError):
        ops.perturbed_linear(x, w, n_pop=2, bm=4)
    with pytest.raises(ValueError):
        ops.perturbed_linear(x, torch.zeros(4, 16, device="cuda"), n_pop=3, bm=4)


@pytest.mark.parametrize("n_pop,bm,k,a,rank,t_steps,first,lif", [
    (16, 16, 64, 16, 8, 1, 0, False),    # a head projection of the transformer
    (16, 16, 64, 64, 8, 1, 2, True),     # output / feed-forward projection, one LIF step, shifted thread ids
    (6, 16, 49, 64, 8, 4, 0, False),     # the encoder: 128 rows per pair in four chunks of 32, k not a multiple of 4
    (4, 3, 20, 10, 4, 2, 4, False),      # 12 rows per pair (partial chunk), ten columns, rank 4
    (2, 1, 5, 3, 16, 1, 0, False),       # tiny everything, rank 16
])
def test_narrow_layer_path_matches_oracle(hs, oracle, n_pop, bm, k, a, rank, t_steps, first, lif):
    """Layers with k, a <= 64 and rank <= 16 take the persistent narrow-layer kernel (algo AUTO):
    same results as the oracle and as the general path, with regenerated and with cached factors."""
    from hyperscalees_b200 import ops, core
    ctx = core.get_context(0)
    g = np.random.default_rng(k * 100 + a)
    x = g.standard_normal((t_steps, n_pop, bm, k)).astype(np.float32)
    w = (g.standard_normal((a, k)) / np.sqrt(k)).astype(np.float32)
    key, sigma = 0x77C0FFEE, 0.4
    kw = dict(n_pop=n_pop, bm=bm, t_steps=t_steps, sigma=sigma, rank=rank, key=key, epoch=2, first_thread=first)
    if lif:
        kw.update(lif=True, tau_m=2.0, v_th=0.1)
    xd, wd = torch.as_tensor(x, device="cuda"), torch.as_tensor(w, device="cuda")
    ctx.profile_enable(True)
    got = ops.perturbed_linear(xd, wd, **kw)
    names = {n for n, v in ctx.profile_read().items() if v[0]}
    ctx.profile_enable(False)
    assert "small_pair" in names
    simt = ops.perturbed_linear(xd, wd, algo=ops.ALGO_SIMT, **kw)
    cache = ops.FactorCache(key, 2, 0, rank, a, k, n_pop // 2, first_pair=first // 2)
    cached = ops.perturbed_linear(xd, wd, cache=cache, **kw)
    assert torch.equal(cached, got)
    if lif:
        assert (got != simt).float().mean().item() <= 1e-3
    else:
        want = np.empty((t_steps * n_pop * bm, a), np.float32)
        for t in range(t_steps):
            for i in range(n_pop):
                r0 = (t * n_pop + i) * bm
                want[r0:r0 + bm] = oracle.do_mm(x[t, i], w, sigma, rank, key, (2, first + i), 0, True)
        scale = max(1.0, np.abs(want).max())
        assert np.abs(got.cpu().numpy() - want).max() <= 2e-5 * scale
        assert (got - simt).abs().max().item() <= 2e-5 * scale
    assert ctx.device_status() == 0
