"""The benchmark configurations at their full sizes, through properties that do not need the CPU
restatement to run the whole workload: sampled members against the oracle, shards against the
whole, cached against regenerated factors, determinism."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

KEY = 0x3C6EF372FE94F82A


def status_ok():
    from hyperscalees_b200 import core
    assert core.get_context(0).device_status() == 0, "a kernel gave up on a bounded wait"


def test_config1_full_size_properties(hs, oracle):
    """Perturbed-linear microbench: x[8192, 16, 1024], W[1024, 1024], rank 16, sigma 0.02, one LIF step."""
    from hyperscalees_b200 import ops
    n_pop, bm, k, a, rank, sigma, tau_m, v_th = 8192, 16, 1024, 1024, 16, 0.02, 20.0, 0.3
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(n_pop, bm, k, device="cuda", generator=g)
    w = torch.randn(a, k, device="cuda", generator=g)
    kw = dict(bm=bm, sigma=sigma, rank=rank, key=KEY, lif=True, tau_m=tau_m, v_th=v_th)
    spikes, pot = ops.perturbed_linear(x, w, n_pop=n_pop, want_potentials=True, **kw)
    status_ok()
    assert set(torch.unique(spikes).tolist()) <= {0.0, 1.0}
    # deterministic
    again = ops.perturbed_linear(x, w, n_pop=n_pop, **kw)
    assert torch.equal(again, spikes)
    # the second half of the population as a shard of its own gives the same rows
    half = n_pop // 2
    shard = ops.perturbed_linear(x[half:], w, n_pop=half, first_thread=half, **kw)
    assert torch.equal(shard, spikes[half * bm:])
    # factors read from a cache give the bits of the regenerated ones
    cache = ops.FactorCache(KEY, 0, 0, rank, a, k, n_pairs=n_pop // 2)
    cached = ops.perturbed_linear(x, w, n_pop=n_pop, cache=cache, **kw)
    assert torch.equal(cached, spikes)
    status_ok()
    # sampled members against the CPU restatement (fp64-accumulated potentials as the yardstick)
    wn = w.cpu().numpy()
    for i in (0, 1, 4097, 8191):
        xi = x[i:i + 1].cpu().numpy()
        want_s = oracle.perturbed_linear_lif(xi, wn, sigma, rank, KEY, first_thread=i, tau_m=tau_m, v_th=v_th)
        _, c64 = oracle.perturbed_linear_lif(xi, wn, sigma, rank, KEY, first_thread=i, tau_m=tau_m, v_th=v_th,
                                             acc64=True, want_potentials=True)
        got_s = spikes[i * bm:(i + 1) * bm].cpu().numpy().reshape(want_s.shape)
        got_c = pot[i * bm:(i + 1) * bm].cpu().numpy().reshape(c64.shape)
        assert np.abs(got_c - c64).max() <= 1e-5 * max(1.0, np.abs(c64).max())
        mism = got_s != want_s
        assert mism.mean() <= 1e-4
        assert (np.abs(c64[mism] - v_th) < 1e-5 * max(1.0, np.abs(c64).max())).all()
    # antithetic partners share the clean product: their potentials differ by twice the rank-r term only
    clean = ops.perturbed_linear(x[:2], w, n_pop=2, bm=bm, perturb=False)
    p0, p1 = pot[:bm] * tau_m, pot[bm:2 * bm] * tau_m
    u0, u1 = p0 - clean[:bm], p1 - clean[bm:]
    assert u0.abs().max().item() > 0
    # same factors with opposite signs applied to different inputs: both corrections are small against the product
    assert u0.abs().max().item() < 0.2 * clean.abs().max().item() and u1.abs().max().item() < 0.2 * clean.abs().max().item()


@pytest.mark.parametrize("rank", [64, 96, 128])
def test_config3_full_size_properties(hs, oracle, rank):
    """Large-population SNN MLP 784-128-128-128-10, T = 8, N = 65 536 members of one sample, at the
    three ranks the configuration sweeps (96 takes the zero-filled last k-block of the tensor-core
    contraction, 64 and 128 whole k-blocks)."""
    from hyperscalees_b200 import models, noiser, ops
    dims, n_pop, bm, T, sigma = [784, 128, 128, 128, 10], 65536, 1, 8, 0.02
    g = np.random.Generator(np.random.PCG64(0))
    img = g.random((n_pop, 784), dtype=np.float32)
    img[g.random((n_pop, 784)) < 0.8] = 0.0
    labels = g.integers(0, 10, n_pop).astype(np.int32)
    di, dl = torch.as_tensor(img, device="cuda"), torch.as_tensor(labels, device="cuda")
    seeds = [1, 2, 3, 4]
    keys = models.default_base_keys(len(dims))

    def fresh(first, n, cache):
        net = models.SnnMlp(dims, tau_m=2.0, v_th=1.0, reset_mode=1, seed=0)
        net.weights = [w * 4.0 for w in net.weights]   # N(0, 1/fan_in) alone leaves the net silent at v_th = 1
        frozen, nz = noiser.init_noiser(net.params(), sigma, 0.01, 0, False, 0, rank, noiser.Solver.adamw(0.01))
        return net, models.PopulationStep(net, frozen, nz, keys, T, n, bm, first_thread=first, cache=cache,
                                          n_total=n_pop if n == n_pop else None)

    net, step = fresh(0, n_pop, "auto")
    raw = step.eval(di, dl, seeds)
    status_ok()
    assert torch.isfinite(raw).all() and raw.std().item() > 0
    assert torch.equal(step.eval(di, dl, seeds), raw)          # deterministic
    om = oracle.Snn([w.cpu().numpy() for w in net.weights], keys, 1.0, 2.0, 1.0, None, 1, sigma, rank, 0)

    def check_members(got, images, lbls, first_thread, count=4):
        # the Poisson stream is indexed by the element's position in the call's own batch
        spk = oracle.poisson_encode(images[:count], T, seeds)
        for j in range(count):
            lg = om.forward(spk[:, j:j + 1], (0, first_thread + j))
            want = oracle.fitness(lg, lbls[j:j + 1])[0]
            assert abs(got[j].item() - want) <= 1e-3 * max(1.0, abs(want))

    check_members(raw, img, labels, 0)
    # a quarter of the population as a shard of its own (thread ids lo..hi), factors regenerated
    # instead of cached: the per-pair path with scratch chunks at full shard size
    lo, hi = n_pop // 2, n_pop // 2 + n_pop // 4
    _, shard = fresh(lo, hi - lo, "off")
    raw_shard = shard.eval(di[lo:hi], dl[lo:hi], seeds)
    status_ok()
    assert torch.isfinite(raw_shard).all()
    check_members(raw_shard, img[lo:hi], labels[lo:hi], lo)
    # the gradient of the first and of a hidden layer at full size, against sub-blocks of the CPU
    # restatement's sum over all 65 536 members (corners and the ragged last column tile included)
    fit = ops.convert_fitnesses(raw)
    # mean and E[x^2] are fp32 sums of 65 536 terms taken in another order than the restatement's loop
    assert np.abs(fit.cpu().numpy() - oracle.convert_fitnesses(raw.cpu().numpy())).max() <= 1e-3
    fit_h = fit.cpu().numpy()
    epochs, tids = np.zeros(n_pop, np.int32), np.arange(n_pop, dtype=np.int32)
    for layer, blocks in ((0, [((0, 6), (0, 6)), ((122, 128), (778, 784)), ((60, 64), (300, 306))]),
                          (2, [((0, 6), (122, 128)), ((100, 104), (0, 6))])):
        a_, b_ = dims[layer + 1], dims[layer]
        grad = ops.es_update(keys[layer], 0, 0, rank, a_, b_, sigma, fit, cache=step.caches[layer])
        regen = ops.es_update(keys[layer], 0, 0, rank, a_, b_, sigma, fit) if layer == 2 else None
        status_ok()
        gmax = grad.abs().max().item()
        assert np.isfinite(gmax) and gmax > 0
        if regen is not None:   # factors regenerated chunk by chunk: same sum, another split of the pairs
            assert (regen - grad).abs().max().item() <= 2e-4 * gmax
        gh = grad.cpu().numpy()
        for rows, cols in blocks:
            want = oracle.lora_grad_block(sigma, keys[layer], a_, b_, rank, fit_h, epochs, tids, rows, cols)
            assert np.abs(gh[rows[0]:rows[1], cols[0]:cols[1]] - want).max() <= 1e-3 * gmax
    before = [p.clone() for p in step.params]
    step.update(raw)
    status_ok()
    for b, a in zip(before[:-1], step.params[:-1]):
        assert torch.isfinite(a).all() and (a - b).abs().max().item() > 0
    # the first layer after the solver step is what one AdamW step on that gradient gives
    grad0 = ops.es_update(keys[0], 0, 0, rank, dims[1], dims[0], sigma, fit, cache=step.caches[0])
    want_p = oracle.solver_update(2, 1, before[0].cpu().numpy(), grad0.cpu().numpy(),
                                  np.zeros_like(grad0.cpu().numpy()), np.zeros_like(grad0.cpu().numpy()),
                                  lr=0.01, weight_decay=1e-4)
    want_p = want_p[0] if isinstance(want_p, tuple) else want_p
    assert np.abs(step.params[0].cpu().numpy() - want_p).max() <= 1e-3 * np.abs(want_p).max()


def test_config2_full_size_sampled_members(hs, oracle):
    """Token-level spiking transformer at BASELINE's size (4096 members x 32 sequences x 64 tokens,
    d_model 64, 4 heads, 2 blocks, vocab 256, rank 8): deterministic, a chunk boundary does not
    change a member's value, sampled members match the CPU composition."""
    from hyperscalees_b200 import models
    from hyperscalees_b200.spiking_lm import LmNoise, SpikingLM
    from oracle import spiking_lm as SL
    vocab, L, d, H, blocks, rank, sigma, n, seqs = 256, 64, 64, 4, 2, 8, 0.02, 4096, 32
    m = SpikingLM(vocab, L, d, H, blocks, mlp_ratio=4, T=4, seed=2)
    g = torch.Generator(device="cuda").manual_seed(2)
    ids = torch.randint(0, vocab, (n, seqs, L), device="cuda", generator=g, dtype=torch.int32)
    keys = models.default_base_keys(len(m.params()))
    noise = LmNoise(sigma, rank, keys)
    fit = m.fitness(ids, noise, chunk_members=1024)
    status_ok()
    assert torch.isfinite(fit).all() and fit.std().item() > 0
    assert torch.equal(m.fitness(ids, noise, chunk_members=1024), fit)
    part = m.fitness(ids[1000:1064].contiguous(), LmNoise(sigma, rank, keys, first_thread=1000), chunk_members=64)
    assert torch.equal(part, fit[1000:1064])
    npm = {"emb": m.emb.cpu().numpy(), "pos_emb": m.pos_emb.cpu().numpy(), "out": m.out.cpu().numpy(),
           "blocks": [{k: ([w.cpu().numpy() for w in v] if isinstance(v, list) else v.cpu().numpy())
                       for k, v in blk.items()} for blk in m.blocks],
           "T": m.T, "tau_m": m.tau_m, "v_th": m.v_th, "beta": m.beta, "num_heads": m.num_heads}
    ih = ids.cpu().numpy()
    for j in (0, 1, 2049, 4095):
        want = SL.member_fitness(SL.member_forward(npm, ih[j], sigma, rank, keys, (0, j)), ih[j])
        assert abs(fit[j].item() - want) <= 1e-3 * max(1.0, abs(want))
