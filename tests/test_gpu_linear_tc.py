"""The tcgen05 path of the perturbed linear layer against the CPU oracle and
against the general fp32 path (same criteria as test_gpu_linear.py)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

KEY = 0x3C6EF372FE94F82A


def dev(a):
    return torch.as_tensor(np.ascontiguousarray(a), device="cuda")


def status_ok():
    from hyperscalees_b200 import core
    assert core.get_context(0).device_status() == 0, "a kernel gave up on a bounded wait"


@pytest.mark.parametrize("n_pop,bm,k,a,rank,t_steps,first", [
    (8, 16, 64, 128, 4, 1, 0),      # one tile, BN = 128
    (16, 16, 256, 256, 16, 1, 0),   # BN = 256, several k-blocks
    (8, 16, 128, 512, 16, 2, 2),    # two N chunks, two time steps, non-zero first member
    (4, 32, 96, 128, 8, 1, 1),      # bm = 32: one member per warp slice, odd first member
    (2, 64, 800, 128, 4, 2, 0),     # SNN-like first layer (k = 800 = 25 k-blocks)
    (40, 16, 64, 384, 4, 1, 0),     # more tiles than one wave would need on a small grid? no: exercises a = 3*128
])
def test_tensor_path_matches_oracle(hs, oracle, n_pop, bm, k, a, rank, t_steps, first):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(n_pop * 100 + k + a)
    x = g.standard_normal((t_steps, n_pop, bm, k)).astype(np.float32)
    w = (g.standard_normal((a, k)) / np.sqrt(k)).astype(np.float32)
    sigma = 0.5
    kw = dict(n_pop=n_pop, bm=bm, t_steps=t_steps, sigma=sigma, rank=rank, key=KEY, epoch=3, first_thread=first,
              noise_reuse=1)
    got = ops.perturbed_linear(dev(x), dev(w), algo=ops.ALGO_TENSOR, **kw).cpu().numpy()
    status_ok()
    want = np.empty_like(got)
    flat = x.reshape(t_steps, n_pop, bm, k)
    for t in range(t_steps):
        for i in range(n_pop):
            r0 = (t * n_pop + i) * bm
            want[r0:r0 + bm] = oracle.do_mm(flat[t, i], w, sigma, rank, KEY, (3, first + i), 1, True)
    scale = max(np.abs(want).max(), 1.0)
    assert np.abs(got - want).max() <= 2e-5 * scale
    simt = ops.perturbed_linear(dev(x), dev(w), algo=ops.ALGO_SIMT, **kw).cpu().numpy()
    assert np.abs(got - simt).max() <= 2e-5 * scale
    clean = ops.perturbed_linear(dev(x), dev(w), n_pop=n_pop, bm=bm, t_steps=t_steps, perturb=False,
                                 algo=ops.ALGO_TENSOR).cpu().numpy()
    status_ok()
    assert np.abs(clean - x.reshape(-1, k).astype(np.float64) @ w.T.astype(np.float64)).max() <= 2e-5 * scale


@pytest.mark.parametrize("tau_m,v_th", [(20.0, 0.3), (2.0, 1.0)])
def test_tensor_path_fused_lif_spikes(hs, oracle, tau_m, v_th):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(7)
    n_pop, bm, k, a, rank = 32, 16, 256, 256, 16
    x = g.standard_normal((n_pop, bm, k)).astype(np.float32)
    w = g.standard_normal((a, k)).astype(np.float32)
    sigma = 0.02
    got_s, got_c = ops.perturbed_linear(dev(x), dev(w), n_pop=n_pop, bm=bm, sigma=sigma, rank=rank, key=KEY,
                                        lif=True, tau_m=tau_m, v_th=v_th, want_potentials=True,
                                        algo=ops.ALGO_TENSOR)
    status_ok()
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


def test_tensor_path_many_tiles_linearity(hs):
    """More M tiles than SMs (persistent loop) at a size the oracle would not finish quickly:
    y(x1 + x2) == y(x1) + y(x2) for the clean product, and the noisy product minus the clean one
    equals the low-rank term computed by the general path."""
    from hyperscalees_b200 import ops
    torch.manual_seed(0)
    n_pop, bm, k, a, rank = 2048, 16, 256, 256, 8   # 256 M tiles
    x1 = torch.randn(n_pop, bm, k, device="cuda")
    x2 = torch.randn(n_pop, bm, k, device="cuda")
    w = torch.randn(a, k, device="cuda")
    kw = dict(n_pop=n_pop, bm=bm, perturb=False, algo=ops.ALGO_TENSOR)
    y12 = ops.perturbed_linear(x1 + x2, w, **kw)
    y1 = ops.perturbed_linear(x1, w, **kw)
    y2 = ops.perturbed_linear(x2, w, **kw)
    status_ok()
    assert (y12 - (y1 + y2)).abs().max().item() <= 2e-4
    kw = dict(n_pop=n_pop, bm=bm, sigma=0.3, rank=rank, key=KEY)
    nt = ops.perturbed_linear(x1, w, algo=ops.ALGO_TENSOR, **kw)
    ns = ops.perturbed_linear(x1, w, algo=ops.ALGO_SIMT, **kw)
    status_ok()
    assert (nt - ns).abs().max().item() <= 2e-5 * ns.abs().max().item()


def test_tensor_path_refuses_unsupported_shapes(hs):
    from hyperscalees_b200 import ops
    from hyperscalees_b200._lib import HsesError
    x = torch.zeros(5 * 3, 40, device="cuda")
    w = torch.zeros(24, 40, device="cuda")
    with pytest.raises(HsesError) as e:
        ops.perturbed_linear(x, w, n_pop=5, bm=3, sigma=0.1, rank=4, key=1, algo=ops.ALGO_TENSOR)
    assert e.value.status == 4
    # AUTO falls back to the general path for the same call
    out = ops.perturbed_linear(x, w, n_pop=5, bm=3, sigma=0.1, rank=4, key=1)
    assert out.shape == (15, 24)


@pytest.mark.parametrize("taper", [False, True])
def test_host_pipeline_equals_single_call(hs, taper):
    """The chunked, stream-overlapped host path gives the same spikes as one device call."""
    from hyperscalees_b200 import ops
    torch.manual_seed(1)
    n_pop, bm, k, a = 128, 16, 128, 256
    x = torch.randn(n_pop, bm, k).pin_memory()
    w = torch.randn(a, k, device="cuda")
    out = torch.empty(n_pop * bm, a).pin_memory()
    kw = dict(sigma=0.05, rank=8, key=KEY, lif=True, tau_m=20.0, v_th=0.3)
    pipe = ops.HostPipeline(n_pop, bm, k, a, chunks=4, taper=taper)
    assert sum(pipe.sizes) == n_pop and all(m % 2 == 0 for m in pipe.sizes)
    assert (len(set(pipe.sizes)) > 1) == taper
    pipe.run(x, w, out, first_thread=6, **kw)
    torch.cuda.synchronize()
    want = ops.perturbed_linear(x.cuda(), w, n_pop=n_pop, bm=bm, first_thread=6, **kw).cpu()
    assert torch.equal(out, want)
    status_ok()


@pytest.mark.parametrize("perturb", [False, True])
def test_tensor_path_with_inputs_exact_in_fp16(hs, oracle, perturb):
    """0/1 spike inputs have an all-zero lo half: the kernel drops that pass.  The result must
    equal the general path's to fp32 rounding, and switching back to inputs with a non-zero lo
    half in the next call must bring the pass back."""
    from hyperscalees_b200 import ops
    g = np.random.default_rng(12)
    n_pop, bm, k, a, rank = 8, 16, 256, 256, 16
    spikes = (g.random((n_pop, bm, k)) < 0.2).astype(np.float32)
    dense = g.standard_normal((n_pop, bm, k)).astype(np.float32)
    w = (g.standard_normal((a, k)) / np.sqrt(k)).astype(np.float32)
    kw = dict(n_pop=n_pop, bm=bm, sigma=0.5, rank=rank, key=KEY, perturb=perturb)
    for x in (spikes, dense, spikes):
        got = ops.perturbed_linear(dev(x), dev(w), algo=ops.ALGO_TENSOR, **kw)
        ref = ops.perturbed_linear(dev(x), dev(w), algo=ops.ALGO_SIMT, **kw)
        scale = max(ref.abs().max().item(), 1.0)
        assert (got - ref).abs().max().item() <= 2e-5 * scale
    status_ok()
