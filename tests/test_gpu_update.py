"""Parity of the fitness-weighted update with the CPU oracle (rtol 1e-3, fp32 accumulate)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

KEY = 0xDAA66D2C7DDF743F


def dev(a):
    return torch.as_tensor(np.ascontiguousarray(a), device="cuda")


@pytest.mark.parametrize("a,b,rank,n,first", [
    (2, 2, 1, 2, 0), (128, 784, 4, 64, 0), (10, 128, 8, 30, 4), (130, 70, 3, 18, 2), (48, 48, 16, 256, 0),
])
def test_es_update_matches_oracle(hs, oracle, a, b, rank, n, first):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(n + a)
    f = g.standard_normal(n).astype(np.float32)
    got = ops.es_update(KEY, 5, 2, rank, a, b, 0.2, dev(f), first_thread=first).cpu().numpy()
    want = oracle.lora_grad(0.2, KEY, a, b, rank, f, [5] * n, list(range(first, first + n)), 2)
    assert np.abs(got - want).max() <= 1e-3 * np.abs(want).max()


def test_es_update_is_deterministic(hs):
    from hyperscalees_b200 import ops
    f = torch.randn(512, device="cuda")
    g1 = ops.es_update(KEY, 0, 0, 8, 64, 96, 0.1, f)
    g2 = ops.es_update(KEY, 0, 0, 8, 64, 96, 0.1, f)
    assert torch.equal(g1, g2)


def test_es_update_shards_sum_to_whole(hs):
    # a population split across ranks: partial gradients with n_total = N add up
    from hyperscalees_b200 import ops
    f = torch.randn(128, device="cuda")
    whole = ops.es_update(KEY, 0, 0, 4, 32, 40, 0.1, f)
    parts = sum(ops.es_update(KEY, 0, 0, 4, 32, 40, 0.1, f[i:i + 32].contiguous(), first_thread=i, n_total=128)
                for i in range(0, 128, 32))
    assert torch.allclose(whole, parts, rtol=1e-4, atol=1e-6)


def test_antithetic_pair_with_equal_fitness_cancels(hs):
    from hyperscalees_b200 import ops
    f = torch.tensor([0.7, 0.7, -1.2, -1.2], device="cuda")
    assert ops.es_update(KEY, 0, 0, 4, 16, 16, 0.3, f).abs().max().item() == 0.0


@pytest.mark.parametrize("shape", [(1, 1), (2, 1), (3, 17)])
def test_es_update_dense_matches_oracle(hs, oracle, shape):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(shape[1])
    n = 40
    f = g.standard_normal(n).astype(np.float32)
    got = ops.es_update_dense(KEY, 1, 0, shape, 0.3, dev(f), first_thread=2).cpu().numpy()
    want = oracle.full_grad(0.3, KEY, shape[0], shape[1], f, [1] * n, list(range(2, 2 + n)), 0)
    assert np.abs(got - want).max() <= 1e-3 * np.abs(want).max() + 1e-7


def test_alteggroll_sign_update_matches_oracle(hs, oracle):
    """AltEggRoll (alteggroll.rs:65-90): the update contracts the sign patterns of the factors."""
    from hyperscalees_b200 import ops
    n, rank, a, b, sigma, key = 48, 4, 18, 30, 0.4, 123
    f = np.random.default_rng(4).standard_normal(n).astype(np.float32)
    want = oracle.alt_lora_grad(sigma, key, a, b, rank, f, [1] * n, list(range(n)), 0)
    ft = torch.from_numpy(f).cuda()
    got = ops.es_update(key, 1, 0, rank, a, b, sigma, ft, sign_factors=True)
    assert np.allclose(got.cpu().numpy(), want, rtol=1e-3, atol=1e-6)
    plain = ops.es_update(key, 1, 0, rank, a, b, sigma, ft)
    assert not torch.equal(plain, got)     # alteggroll.rs:252-266: differs from EggRoll's update
    cache = ops.FactorCache(key, 1, 0, rank, a, b, n // 2)
    assert torch.equal(ops.es_update(key, 1, 0, rank, a, b, sigma, ft, cache=cache, sign_factors=True), got)


def test_alteggroll_noiser_mirror(hs, oracle):
    from hyperscalees_b200 import noiser
    p = torch.zeros(2, 2, device="cuda")
    frozen, nz = noiser.init_noiser([p], 0.5, 0.1, 0, False, 0, 1, noiser.Solver.sgd(0.1))
    fit = torch.tensor([1.0, 0.0], device="cuda")
    infos = [noiser.IterInfo(0, 0), noiser.IterInfo(0, 1)]
    (g,) = noiser.AltEggRoll().grads(frozen, nz, [p], [7], fit, infos, [noiser.MM_PARAM])
    # alteggroll.rs:205-243 with N = 2: entries are -(sigma/sqrt(r)) * sign(a_i) * sign(b_j) / N * sqrt(N)
    A, B = oracle.lora_params(1.0, 7, 1, 0, 0, 2, 2, 0)
    want = -(0.5 * np.sign(A) @ np.sign(B).T) / 2 * np.sqrt(2.0)
    assert np.allclose(g.cpu().numpy(), want, rtol=1e-5)


@pytest.mark.parametrize("a,b,rank,n,first", [
    (128, 784, 64, 64, 0),      # config-3 first layer: 4 column tiles of 208 (the last one ragged)
    (128, 128, 128, 40, 4),     # two k-blocks per pair
    (256, 136, 64, 8, 0),       # two row tiles, fewer pairs than the split count would like
    (128, 16, 64, 2, 0),        # a single pair, the narrowest tile
    (10, 128, 64, 24, 0),       # readout layer: fewer rows than one tile
    (130, 70, 64, 6, 2),        # ragged in both directions
    (128, 784, 96, 16, 0),      # rank 96: the second k-block of a pair is half zero fill
    (40, 50, 48, 10, 2),        # rank 48: one k-block, three quarters full
    (128, 128, 160, 6, 0),      # rank 160: three k-blocks, the last one half full
])
def test_tensor_core_update_matches_oracle_and_general_kernel(hs, oracle, a, b, rank, n, first):
    """The tcgen05 contraction of the update against the oracle and against the fp32 kernel."""
    from hyperscalees_b200 import ops
    g = np.random.default_rng(a + b + n)
    f = (g.standard_normal(n) * 3).astype(np.float32)
    kw = dict(first_thread=first)
    got = ops.es_update(KEY, 5, 2, rank, a, b, 0.2, dev(f), algo=ops.ALGO_TENSOR, **kw)
    general = ops.es_update(KEY, 5, 2, rank, a, b, 0.2, dev(f), algo=ops.ALGO_SIMT, **kw)
    want = oracle.lora_grad(0.2, KEY, a, b, rank, f, [5] * n, list(range(first, first + n)), 2)
    scale = np.abs(want).max()
    assert np.abs(got.cpu().numpy() - want).max() <= 1e-3 * scale
    assert (got - general).abs().max().item() <= 2e-5 * scale      # three fp16 passes are fp32-equivalent
    cache = ops.FactorCache(KEY, 5, 2, rank, a, b, n // 2, first // 2)
    assert torch.equal(ops.es_update(KEY, 5, 2, rank, a, b, 0.2, dev(f), cache=cache, algo=ops.ALGO_TENSOR, **kw), got)
    # deterministic, raw accumulation and the sign variant go through the same kernels
    assert torch.equal(ops.es_update(KEY, 5, 2, rank, a, b, 0.2, dev(f), algo=ops.ALGO_TENSOR, **kw), got)
    acc = torch.ones(a, b, device="cuda")
    ops.es_update(KEY, 5, 2, rank, a, b, 0.2, dev(f), out=acc, mode=ops.UPDATE_RAW_ACC, algo=ops.ALGO_TENSOR, **kw)
    ref = torch.ones(a, b, device="cuda")
    ops.es_update(KEY, 5, 2, rank, a, b, 0.2, dev(f), out=ref, mode=ops.UPDATE_RAW_ACC, algo=ops.ALGO_SIMT, **kw)
    assert (acc - ref).abs().max().item() <= 2e-5 * (ref - 1).abs().max().item()
    s_tc = ops.es_update(KEY, 5, 2, rank, a, b, 0.2, dev(f), sign_factors=True, algo=ops.ALGO_TENSOR, **kw)
    s_ref = ops.es_update(KEY, 5, 2, rank, a, b, 0.2, dev(f), sign_factors=True, algo=ops.ALGO_SIMT, **kw)
    assert (s_tc - s_ref).abs().max().item() <= 2e-5 * s_ref.abs().max().item()


def test_tensor_core_update_tiny_and_huge_weights(hs):
    """The weight scale is a power of two found on the device: very small and very large raw
    scores must neither underflow nor overflow the fp16 operands."""
    from hyperscalees_b200 import ops
    for mag in (1e-6, 1.0, 3e4):
        f = torch.randn(32, device="cuda") * mag
        tc = ops.es_update(KEY, 0, 0, 64, 128, 64, 0.1, f, algo=ops.ALGO_TENSOR)
        ref = ops.es_update(KEY, 0, 0, 64, 128, 64, 0.1, f, algo=ops.ALGO_SIMT)
        assert torch.isfinite(tc).all()
        assert (tc - ref).abs().max().item() <= 2e-5 * ref.abs().max().item()
    z = ops.es_update(KEY, 0, 0, 64, 128, 64, 0.1, torch.zeros(32, device="cuda"), algo=ops.ALGO_TENSOR)
    assert torch.count_nonzero(z).item() == 0
