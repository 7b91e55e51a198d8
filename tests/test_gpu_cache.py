"""The device-resident factor cache (LoraNoiseCache, eggroll.rs:229-309): cached calls must
return the same bits as calls that regenerate the factors, and the chunked raw accumulation
(accumulated_update_cached, eggroll.rs:577-702) must reproduce the one-shot gradient."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ops():
    from hyperscalees_b200 import ops
    return ops


def test_cache_holds_the_oracle_normals():
    ops = _ops()
    from oracle import oracle
    key, rank, a, b = 77, 4, 6, 10
    c = ops.FactorCache(key, epoch=5, noise_reuse=2, rank=rank, a=a, b=b, n_pairs=3, first_pair=4)
    for p in range(3):
        # member 2*(4+p) has sign +1: its A is the raw block times base_sigma = 1
        A, B = oracle.lora_params(1.0, key, rank, 5, 2 * (4 + p), a, b, 2)
        assert np.array_equal(c.A[p].cpu().numpy(), A)
        assert np.array_equal(c.B[p].cpu().numpy(), B)


@pytest.mark.parametrize("shape", [
    dict(n_pop=6, bm=3, k=20, a=9, rank=3, first=4),          # general path
    dict(n_pop=64, bm=16, k=128, a=256, rank=16, first=0),    # tensor path, 256-column chunks
    dict(n_pop=16, bm=32, k=64, a=128, rank=4, first=2),      # tensor path, 128-column chunks
])
def test_linear_with_cache_is_bit_equal(shape):
    ops = _ops()
    n_pop, bm, k, a, rank, first = (shape[s] for s in ("n_pop", "bm", "k", "a", "rank", "first"))
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(n_pop, bm, k, device="cuda", generator=g)
    w = torch.randn(a, k, device="cuda", generator=g)
    kw = dict(n_pop=n_pop, bm=bm, sigma=0.3, rank=rank, key=99, epoch=7, first_thread=first, noise_reuse=3)
    ref = ops.perturbed_linear(x, w, **kw)
    first_pair = first // 2
    n_pairs = (first + n_pop - 1) // 2 - first_pair + 1
    # a cache that starts earlier and ends later than the call needs
    c = ops.FactorCache(99, epoch=7, noise_reuse=3, rank=rank, a=a, b=k, n_pairs=n_pairs + 3,
                        first_pair=max(first_pair - 1, 0))
    got = ops.perturbed_linear(x, w, cache=c, **kw)
    assert torch.equal(ref, got)
    spikes_ref = ops.perturbed_linear(x, w, lif=True, tau_m=2.0, v_th=0.5, **kw)
    spikes = ops.perturbed_linear(x, w, lif=True, tau_m=2.0, v_th=0.5, cache=c, **kw)
    assert torch.equal(spikes_ref, spikes)


def test_cache_is_checked_against_the_call():
    ops = _ops()
    from hyperscalees_b200._lib import HsesError
    x = torch.randn(4, 2, 8, device="cuda")
    w = torch.randn(5, 8, device="cuda")
    c = ops.FactorCache(1, epoch=0, noise_reuse=0, rank=2, a=5, b=8, n_pairs=2)
    kw = dict(n_pop=4, bm=2, sigma=0.1, rank=2, cache=c)
    ops.perturbed_linear(x, w, key=1, **kw)
    with pytest.raises(HsesError):
        ops.perturbed_linear(x, w, key=2, **kw)                       # another parameter
    with pytest.raises(HsesError):
        ops.perturbed_linear(x, w, key=1, epoch=3, noise_reuse=1, **kw)  # another epoch bucket
    with pytest.raises(HsesError):
        ops.perturbed_linear(x, w, key=1, first_thread=2, **kw)       # members beyond the cache


def test_update_with_cache_matches_regeneration():
    ops = _ops()
    n, rank, a, b = 64, 4, 20, 36
    f = torch.randn(n, device="cuda")
    ref = ops.es_update(5, 0, 0, rank, a, b, 0.2, f)
    c = ops.FactorCache(5, 0, 0, rank, a, b, n_pairs=n // 2)
    got = ops.es_update(5, 0, 0, rank, a, b, 0.2, f, cache=c)
    assert torch.equal(ref, got)


def test_chunked_raw_accumulation_equals_one_shot_gradient():
    """accumulated_update (eggroll.rs:550-702): per-chunk sums of raw scores, combined with
    the mean and std of all scores afterwards, give the gradient of the one-shot update."""
    ops = _ops()
    from hyperscalees_b200 import noiser
    n, rank, a, b, sigma = 96, 4, 12, 28, 0.25
    raw = torch.randn(n, device="cuda") * 3 + 1
    fit = ops.convert_fitnesses(raw, 0)
    one_shot = ops.es_update(9, 0, 0, rank, a, b, sigma, fit)
    c = ops.FactorCache(9, 0, 0, rank, a, b, n_pairs=n // 2)
    acc = torch.zeros(a, b, device="cuda")
    for lo in range(0, n, 32):
        ops.es_update(9, 0, 0, rank, a, b, sigma, raw[lo:lo + 32].contiguous(), first_thread=lo,
                      out=acc, cache=c, mode=ops.UPDATE_RAW_ACC)
    ones = torch.zeros_like(acc)   # sum of A_i B_i^T over whole antithetic pairs is exactly zero
    r = raw.double()
    mean = float(r.mean())
    std = float(torch.sqrt((r * r).mean() - r.mean() ** 2 + 1e-5))
    (combined,) = noiser.combine_affine_grads([acc], [ones], mean, std, n)
    torch.testing.assert_close(combined, one_shot, rtol=1e-3, atol=1e-5)


def test_population_step_with_caches_is_bit_equal():
    """eval() and update() that read the factor caches give the bits of the regenerating step."""
    from hyperscalees_b200 import models, noiser
    dims, n_pop, bm, T, rank, sigma, lr = [784, 128, 128, 10], 32, 4, 8, 4, 0.1, 0.05
    rng = np.random.default_rng(5)
    img = torch.from_numpy(rng.random((n_pop * bm, 784), dtype=np.float32)).cuda()
    labels = torch.from_numpy(rng.integers(0, 10, n_pop * bm, dtype=np.int32)).cuda()
    keys = models.default_base_keys(len(dims))
    seeds = [3, 1, 4, 1]
    results = []
    for cached in (False, True):
        net = models.SnnMlp(dims, tau_m=1.0, v_th=0.3, seed=2)
        frozen, nz = noiser.init_noiser(net.params(), sigma, lr, 0, False, 0, rank, noiser.Solver.adamw(lr))
        step = models.PopulationStep(net, frozen, nz, keys, T, n_pop, bm)
        if cached:
            held = step.build_caches(epoch=0, n_total=n_pop)
            assert held == sum((a + b) * rank * (n_pop // 2) * 4 for a, b in ((128, 784), (128, 128), (10, 128)))
        raw = step.eval(img, labels, seeds)
        step.update(raw)
        results.append((raw, [p.clone() for p in step.params]))
    assert torch.equal(results[0][0], results[1][0])
    for p0, p1 in zip(results[0][1], results[1][1]):
        assert torch.equal(p0, p1)


def test_population_step_auto_cache_follows_the_epoch_bucket():
    """cache='auto' rebuilds the factor caches exactly when the epoch bucket changes and gives
    the bits of the regenerating step in every epoch."""
    from hyperscalees_b200 import models, noiser
    dims, n_pop, bm, T, rank = [784, 128, 10], 16, 2, 4, 8
    rng = np.random.default_rng(6)
    img = torch.from_numpy(rng.random((n_pop * bm, 784), dtype=np.float32)).cuda()
    labels = torch.from_numpy(rng.integers(0, 10, n_pop * bm, dtype=np.int32)).cuda()
    keys = models.default_base_keys(len(dims))
    net = models.SnnMlp(dims, tau_m=1.0, v_th=0.3, seed=4)
    frozen, nz = noiser.init_noiser(net.params(), 0.2, 0.01, 0, False, 2, rank, noiser.Solver.sgd(0.01))
    plain = models.PopulationStep(net, frozen, nz, keys, T, n_pop, bm)
    auto = models.PopulationStep(net, frozen, nz, keys, T, n_pop, bm, cache="auto", n_total=n_pop)
    seen = []
    for epoch in range(4):                       # noise_reuse = 2: buckets 0, 0, 1, 1
        want = plain.eval(img, labels, [1, 2, 3, 4], epoch=epoch)
        got = auto.eval(img, labels, [1, 2, 3, 4], epoch=epoch)
        assert torch.equal(want, got)
        seen.append(auto.caches[0].data.data_ptr() if auto.caches else None)
        assert auto.caches[0].desc.true_epoch == epoch // 2
    assert seen[0] == seen[1] and seen[2] == seen[3]   # not rebuilt inside a bucket
