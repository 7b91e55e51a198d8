"""The per-pair path of the perturbed linear layer (few rows per antithetic pair, wide
factors — the one-sample-per-member, rank 64..128 configuration) against the CPU oracle,
against the general path, and with a factor cache."""
import numpy as np
import pytest
import torch

from test_gpu_linear import KEY, dev, oracle_mm

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_pop,bm,k,a,rank,t_steps,first", [
    (8, 1, 784, 128, 64, 8, 0),     # config-3 first layer: 16 rows per pair, tensor-core base product
    (6, 1, 128, 10, 96, 1, 2),      # readout: one step, a < 32, rank that does not divide 256
    (4, 2, 36, 50, 8, 3, 4),        # 12 rows per pair, general base product
    (2, 16, 64, 40, 128, 1, 0),     # 32 rows per pair, rank 128
    (4, 1, 20, 1100, 8, 2, 0),      # more output column groups than threads, A too large for shared memory
    (6, 1, 128, 200, 32, 8, 0),     # swizzled A: four column blocks (two rounds of warp tasks), ragged last block
    (4, 4, 64, 100, 64, 2, 2),      # swizzled A, 16 rows per pair, a not a multiple of 8
    (2, 2, 40, 256, 32, 8, 0),      # swizzled A, 32 rows per pair, the largest box (256 rows)
    (4, 3, 64, 72, 32, 2, 0),       # swizzled A, 12 of 16 tile rows used, ragged column block
    (6, 1, 32, 10, 64, 1, 4),       # swizzled A, 2 of 8 tile rows, ten columns (one warp task pair)
    (6, 1, 128, 128, 64, 8, 2),     # config-3 hidden layer, shard offset
    (4, 1, 64, 128, 32, 3, 0),      # the same with 6 of 8 tile rows
    (4, 2, 96, 256, 96, 8, 0),      # 256 outputs, 32 rows per pair, three rank boxes
    (4, 1, 64, 128, 128, 8, 0),     # rank 128
])
def test_pair_path_matches_oracle(hs, oracle, n_pop, bm, k, a, rank, t_steps, first):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(n_pop * 10 + k)
    x = g.standard_normal((t_steps, n_pop, bm, k)).astype(np.float32)
    w = (g.standard_normal((a, k)) / np.sqrt(k)).astype(np.float32)
    kw = dict(n_pop=n_pop, bm=bm, t_steps=t_steps, sigma=0.5, rank=rank, key=KEY, epoch=3,
              first_thread=first, noise_reuse=1)
    got = ops.perturbed_linear(dev(x), dev(w), algo=ops.ALGO_PAIR, **kw)
    want = oracle_mm(oracle, x, w, 0.5, rank, KEY, 3, first, 1, acc64=True)
    scale = max(np.abs(want).max(), 1.0)
    assert np.abs(got.cpu().numpy() - want).max() <= 2e-5 * scale
    general = ops.perturbed_linear(dev(x), dev(w), algo=ops.ALGO_SIMT, **kw)
    assert (got - general).abs().max().item() <= 2e-5 * scale
    # the factor cache gives the same bits as regenerating into scratch
    first_pair = first // 2
    cache = ops.FactorCache(KEY, 3, 1, rank, a, k, n_pairs=n_pop // 2 + 1, first_pair=first_pair)
    cached = ops.perturbed_linear(dev(x), dev(w), algo=ops.ALGO_PAIR, cache=cache, **kw)
    assert torch.equal(cached, got)


def test_pair_path_gain_and_fused_lif(hs, oracle):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(1)
    n_pop, bm, k, a, rank = 6, 2, 48, 24, 16
    x = g.standard_normal((n_pop, bm, k)).astype(np.float32)
    w = (g.standard_normal((a, k)) / np.sqrt(k)).astype(np.float32)
    kw = dict(n_pop=n_pop, bm=bm, sigma=0.3, rank=rank, key=KEY)
    plain = ops.perturbed_linear(dev(x), dev(w), algo=ops.ALGO_PAIR, **kw)
    scaled = ops.perturbed_linear(dev(x), dev(w), algo=ops.ALGO_PAIR, out_scale=2.5, **kw)
    assert torch.equal(scaled, plain * 2.5)
    spikes, pot = ops.perturbed_linear(dev(x), dev(w), algo=ops.ALGO_PAIR, lif=True, tau_m=2.0, v_th=0.2,
                                       want_potentials=True, **kw)
    assert torch.equal(pot, plain * 0.5)
    assert torch.equal(spikes, (pot >= 0.2).float())


def test_auto_dispatch_prefers_the_pair_path(hs):
    """One sample per member and rank 64 must not fall back to the general path."""
    from hyperscalees_b200 import ops, core
    ctx = core.get_context(0)
    x = torch.randn(8, 16, 1, 128, device="cuda")
    w = torch.randn(128, 128, device="cuda")
    ctx.profile_enable(False)
    ops.perturbed_linear(x, w, n_pop=16, bm=1, t_steps=8, sigma=0.1, rank=64, key=1)
    names = {k for k, v in ctx.profile_read().items() if v[0]}
    assert "pair_lowrank" in names and "linear_tc" in names and "lowrank_project" not in names
    from hyperscalees_b200._lib import HsesError
    with pytest.raises(HsesError):
        ops.perturbed_linear(torch.randn(4, 64, 16, device="cuda"), torch.randn(8, 16, device="cuda"),
                             n_pop=4, bm=64, sigma=0.1, rank=4, key=1, algo=ops.ALGO_PAIR)


@pytest.mark.parametrize("n_pop,bm,k,a,rank,t_steps,reset", [
    (8, 1, 784, 128, 64, 8, 0),     # per-pair path, scan inside the kernel (swizzled A)
    (6, 2, 64, 100, 32, 4, 1),      # the same with a ragged column block and the subtractive reset
    (4, 1, 36, 50, 8, 3, 0),        # per-pair path without the swizzled form: currents scanned in place
    (8, 16, 64, 128, 4, 2, 0),      # tensor path: currents scanned in place
    (4, 2, 64, 128, 32, 8, 1),      # two samples per member, subtractive reset
    (4, 1, 96, 256, 64, 4, 0),      # 256 outputs, 8 rows per pair
    (6, 1, 128, 128, 64, 3, 0),     # 6 of 8 tile rows
])
def test_fused_lif_scan_equals_linear_then_scan(n_pop, bm, k, a, rank, t_steps, reset):
    """lif = 2 (LIF scan over the steps fused behind the layer) gives the bits of the two-call form."""
    from hyperscalees_b200 import ops, core
    g = np.random.default_rng(n_pop + k)
    x = torch.as_tensor((g.random((t_steps, n_pop, bm, k)) < 0.3).astype(np.float32), device="cuda")
    w = torch.as_tensor((g.standard_normal((a, k)) * 3.0 / np.sqrt(k)).astype(np.float32), device="cuda")
    kw = dict(n_pop=n_pop, bm=bm, t_steps=t_steps, sigma=0.3, rank=rank, key=0x51ED, epoch=1, tau_m=2.0, v_th=0.5,
              reset_mode=reset)
    cur = ops.perturbed_linear(x, w, **kw)
    want = ops.lif_scan(cur.view(t_steps, n_pop * bm, a), 2.0, 0.5, reset_mode=reset)
    got = ops.perturbed_linear(x, w, lif=2, **kw)
    assert core.get_context(0).device_status() == 0
    assert 0.02 < want.mean().item() < 0.98
    assert torch.equal(got.view_as(want), want)


@pytest.mark.parametrize("n_pop,bm,k,a,rank,t_steps,algo", [
    (8, 1, 128, 128, 64, 8, "auto"),    # per-pair kernel with the scan inside: writes the fp16 copy itself
    (4, 1, 36, 48, 8, 3, "auto"),       # per-pair path without the fused scan: one conversion pass
    (8, 16, 64, 128, 4, 2, "auto"),     # tensor path: scan in place, then the conversion pass
])
def test_out_half_is_the_spikes_and_feeds_the_next_layer(n_pop, bm, k, a, rank, t_steps, algo):
    """out_half receives the layer's spikes as fp16; handed to the next layer as x_half it gives the
    bits that layer computes from the f32 spikes."""
    from hyperscalees_b200 import ops
    g = np.random.default_rng(n_pop + a)
    x = torch.as_tensor((g.random((t_steps, n_pop, bm, k)) < 0.3).astype(np.float32), device="cuda")
    w = torch.as_tensor((g.standard_normal((a, k)) * 3.0 / np.sqrt(k)).astype(np.float32), device="cuda")
    kw = dict(n_pop=n_pop, bm=bm, t_steps=t_steps, sigma=0.3, rank=rank, key=0x51ED, epoch=1, tau_m=2.0, v_th=0.5)
    rows = t_steps * n_pop * bm
    half = torch.full((rows, a), 7.0, dtype=torch.float16, device="cuda")
    spikes = ops.perturbed_linear(x, w, lif=2, out_half=half, **kw)
    plain = ops.perturbed_linear(x, w, lif=2, **kw)
    assert torch.equal(spikes, plain)
    assert torch.equal(half.float(), spikes)
    w2 = torch.as_tensor((g.standard_normal((128, a)) * 2.0 / np.sqrt(a)).astype(np.float32), device="cuda")
    kw2 = dict(kw, key=0x77)
    nxt = ops.perturbed_linear(spikes, w2, lif=2, **kw2)
    nxt_h = ops.perturbed_linear(spikes, w2, lif=2, x_half=half, **kw2)
    assert torch.equal(nxt, nxt_h)
