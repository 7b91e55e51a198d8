"""Bit-exact parity of the Poisson and LIF kernels, tolerance parity of the
fitness / z-score / solver kernels, against the CPU oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.as_tensor(np.ascontiguousarray(a), device="cuda")


@pytest.mark.parametrize("batch,in_dim,pitch", [(1, 1, 1), (3, 784, 784), (5, 784, 832), (7, 13, 13), (4, 100, 128)])
@pytest.mark.parametrize("T", [1, 4, 8])
def test_poisson_bit_exact(hs, oracle, batch, in_dim, pitch, T):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(batch * 1000 + in_dim)
    probs = np.zeros((batch, pitch), np.float32)
    vals = g.random((batch, in_dim), dtype=np.float32)
    vals[g.random((batch, in_dim)) < 0.5] = 0.0
    probs[:, :in_dim] = vals
    seeds = [11, 0xDEADBEEF, 7, 2**32 - 1]
    want = oracle.poisson_encode_pitched(probs, in_dim, T, seeds)[:, :, :in_dim]
    got = ops.poisson_encode(dev(probs)[:, :in_dim], T, seeds)
    assert torch.equal(got.cpu(), torch.from_numpy(want))


def test_poisson_edge_probabilities(hs, oracle):
    from hyperscalees_b200 import ops
    probs = np.array([[0.0, 1.0, -0.5, 1.5, np.nan, 1.1920929e-07, 0.99999994, 0.5]], np.float32)
    want = oracle.poisson_encode(probs, 8, [1, 2, 3, 4])
    got = ops.poisson_encode(dev(probs), 8, [1, 2, 3, 4])
    assert torch.equal(got.cpu(), torch.from_numpy(want))
    assert got[:, 0, 0].sum() == 0 and got[:, 0, 1].sum() == 8


def test_poisson_threshold_sweep(hs, oracle):
    # probabilities placed on and next to representable quotient values
    from hyperscalees_b200 import ops
    ks = np.array([1, 2, 3, 1000, 4194304, 4194305, 8388607, 8388608], np.float32)
    u = (ks / np.float32(8388609.0)).astype(np.float32)
    probs = np.concatenate([u, np.nextafter(u, np.float32(2)), np.nextafter(u, np.float32(-1))])[None, :]
    probs = np.repeat(probs, 64, axis=0)
    want = oracle.poisson_encode(probs, 8, [5, 6, 7, 8])
    got = ops.poisson_encode(dev(probs), 8, [5, 6, 7, 8])
    assert torch.equal(got.cpu(), torch.from_numpy(want))


def test_poisson_rate_tracks_probability(hs):
    # hyperscalees-envs/src/snn_mnist.rs:314-331 asserts the firing rate follows p
    from hyperscalees_b200 import ops
    for p in (0.25, 0.5, 0.75):
        probs = torch.full((4096, 64), p, device="cuda")
        rate = ops.poisson_encode(probs, 8, [1, 2, 3, 4]).mean().item()
        assert abs(rate - p) < 0.01


@pytest.mark.parametrize("T,n,h,pitch", [(1, 1, 1, 1), (8, 33, 128, 128), (8, 17, 100, 128), (5, 3, 7, 7)])
@pytest.mark.parametrize("reset", [0, 1])
@pytest.mark.parametrize("with_v0", [False, True])
def test_lif_scan_bit_exact(hs, oracle, T, n, h, pitch, reset, with_v0):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(T * 100 + n)
    cur = np.zeros((T, n, pitch), np.float32)
    cur[:, :, :h] = (g.standard_normal((T, n, h)) * 3).astype(np.float32)
    v0 = (g.standard_normal((n, h)) * 0.2).astype(np.float32) if with_v0 else np.zeros((n, h), np.float32)
    want_s, want_v = oracle.run_lif(cur[:, :, :h], v0, 20.0, 0.3, reset)
    v = None
    if with_v0:
        vbuf = torch.zeros((n, pitch), device="cuda")
        vbuf[:, :h] = dev(v0)
        v = vbuf[:, :h]
    got = ops.lif_scan(dev(cur)[:, :, :h], 20.0, 0.3, v=v, reset_mode=reset)
    assert torch.equal(got.cpu(), torch.from_numpy(want_s))
    if with_v0:
        assert np.array_equal(v.cpu().numpy().view(np.uint32), want_v.view(np.uint32))


@pytest.mark.parametrize("h,pitch", [(128, 128), (100, 128), (7, 7)])
def test_lif_scan_in_place_equals_out_of_place(hs, h, pitch):
    """cur == spikes is allowed (the fallback of the fused LIF scan uses it): both the
    16-byte-vector kernel (h, pitch multiples of 4) and the scalar one."""
    from hyperscalees_b200 import ops
    g = np.random.default_rng(h)
    buf = torch.zeros((8, 19, pitch), device="cuda")
    buf[:, :, :h] = dev((g.standard_normal((8, 19, h)) * 3).astype(np.float32))
    cur = buf[:, :, :h]
    want = ops.lif_scan(cur, 20.0, 0.3).clone()
    got = ops.lif_scan(cur, 20.0, 0.3, out=cur)
    assert got.data_ptr() == cur.data_ptr()
    assert torch.equal(got, want)


def test_lif_reference_cases(hs):
    # hyperscalees-models/src/snn.rs:707-742
    from hyperscalees_b200 import models
    z = torch.zeros(1, device="cuda")
    assert models.lif_step(20.0, 0.3, z, torch.tensor([10.0], device="cuda"))[1].item() == 1.0
    assert models.lif_step(20.0, 0.3, z, torch.tensor([0.1], device="cuda"))[1].item() == 0.0
    v, fired = z, False
    for _ in range(10):
        v, s = models.lif_step(20.0, 0.3, v, torch.tensor([6.0], device="cuda"))
        fired = fired or s.item() == 1.0
    assert fired
    sp = models.run_lif(models.LifParams(20.0, 0.3), torch.full((4, 1, 2), -10.0, device="cuda"),
                        torch.zeros(1, 2, device="cuda"))
    assert sp.sum().item() == 0


def test_lif_linear_regime_trick(hs, oracle):
    # v_th = -1e9 makes every neuron fire (docs/snn_es_burn_gpu_optimization.md:217-222)
    from hyperscalees_b200 import ops
    cur = torch.randn(3, 5, 8, device="cuda")
    assert ops.lif_scan(cur, 20.0, -1e9).min().item() == 1.0


def test_time_mean(hs):
    from hyperscalees_b200 import ops
    x = (torch.rand(8, 37, 50, device="cuda") < 0.3).float()
    got = ops.time_mean(x)
    assert torch.equal(got, x.sum(0) / 8)


def test_fitness_parity(hs, oracle):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(1)
    logits = (g.standard_normal((1000, 10)) * 4).astype(np.float32)
    labels = g.integers(0, 10, 1000).astype(np.int32)
    for reward in (0, 1):
        got = ops.fitness(dev(logits), dev(labels), reward).cpu().numpy()
        want = oracle.fitness(logits, labels, reward)
        assert np.allclose(got, want, atol=1e-5, rtol=1e-5)
    # reference case with an out-of-range label under the binary reward (snn_mnist.rs:341-356)
    lg = np.array([[1.0, 2.0, 0.5], [3.0, 1.0, 2.0], [0.5, 0.5, 9.0]], np.float32)
    got = ops.fitness(dev(lg), dev(np.array([1, 0, 9], np.int32)), 1).cpu().tolist()
    assert got == [1.0, 1.0, 0.0]


def test_member_mean(hs):
    from hyperscalees_b200 import ops
    x = torch.randn(7 * 5, device="cuda")
    assert torch.allclose(ops.member_mean(x, 7, 5), x.view(7, 5).mean(1), atol=1e-6)


@pytest.mark.parametrize("n,gs", [(4, 0), (4, 2), (256, 0), (65536, 0), (1000, 10), (1, 0)])
def test_convert_fitnesses_parity(hs, oracle, n, gs):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(n)
    raw = (g.standard_normal(n) * 2 - 1.5).astype(np.float32)
    got, stats = ops.convert_fitnesses(dev(raw), gs, want_stats=True)
    want = oracle.convert_fitnesses(raw, gs)
    assert np.allclose(got.cpu().numpy(), want, atol=2e-4, rtol=1e-4)
    assert abs(stats[0].item() - raw.astype(np.float64).mean()) < 1e-4


def test_convert_fitnesses_reference_group_case(hs):
    from hyperscalees_b200 import ops
    out = ops.convert_fitnesses(torch.tensor([1.0, 2.0, 3.0, 4.0], device="cuda"), 2).cpu().numpy()
    e = 0.5 / 1.11803399
    assert np.allclose(out, [-e, e, -e, e], atol=1e-4)


@pytest.mark.parametrize("kind", [0, 1, 2])
def test_solver_parity(hs, oracle, kind):
    from hyperscalees_b200 import ops
    g = np.random.default_rng(kind)
    p = g.standard_normal((13, 17)).astype(np.float32)
    m = np.zeros_like(p)
    v = np.zeros_like(p)
    dp, dm, dv = dev(p).clone(), dev(m).clone(), dev(v).clone()
    for step in range(1, 4):
        grad = g.standard_normal(p.shape).astype(np.float32)
        p, m, v = oracle.solver_update(kind, step, p, grad, m, v, lr=0.01, weight_decay=1e-4 if kind == 2 else 0.0)
        ops.solver_step(kind, step, dp, dev(grad), dm, dv, lr=0.01, weight_decay=1e-4 if kind == 2 else 0.0)
        assert np.allclose(dp.cpu().numpy(), p, atol=1e-6, rtol=1e-6)


def test_prng_normal_half_matches_oracle(hs, oracle):
    """Hybrid Tausworthe half-noise stream (hyperscalees-kernels/src/lib.rs:26-143): the integer
    stream is exact, so every value agrees with the CPU restatement up to the device's
    ln/sqrt/cos/sin (a few ulp of values up to ~6); moments as in the reference's own check."""
    import torch
    from hyperscalees_b200 import kernels
    threads, seeds = 300, (11, 22, 33, 44)
    out = torch.empty(threads * 128, device="cuda")
    kernels.prng_normal_half(out, 0.5, 2.0, seeds)
    got = out.cpu().numpy()
    want = oracle.prng_normal_half(threads, 0.5, 2.0, seeds)
    assert np.abs(got - want).max() <= 2e-5
    assert (got == want).mean() > 0.5
    z = (got - 0.5) / 2.0
    assert abs(z.mean()) < 0.02 and abs(z.std() - 1.0) < 0.02
    with pytest.raises(ValueError):
        kernels.prng_normal_half(torch.empty(100, device="cuda"), 0.0, 1.0, seeds)


def test_poisson_encode_dual_writes_the_same_spikes_as_fp16(hs):
    """hses_poisson_encode_dual through the C ABI: the fp16 copy equals the f32 spikes, and the
    tensor-core layer fed with it (x_half) returns what it returns from the f32 spikes alone."""
    import ctypes as C
    from hyperscalees_b200 import _lib, core, ops
    L = _lib.load()
    ctx = core.get_context(0)
    g = torch.Generator(device="cuda").manual_seed(3)
    batch, in_dim, T = 256, 784, 4
    probs = torch.rand(batch, in_dim, device="cuda", generator=g)
    out = torch.empty(T, batch, in_dim, device="cuda")
    half = torch.empty(T, batch, in_dim, device="cuda", dtype=torch.float16)
    sd = (C.c_uint32 * 4)(1, 2, 3, 4)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.hses_poisson_encode_dual(ctx.handle, stream, C.c_void_p(probs.data_ptr()), batch, in_dim, in_dim, T, sd,
                                    C.c_void_p(out.data_ptr()), C.c_void_p(half.data_ptr()))
    assert rc == 0, L.hses_last_error()
    assert torch.equal(out, ops.poisson_encode(probs, T, [1, 2, 3, 4]))
    assert torch.equal(half.float(), out)
    # clean tensor-core product with and without the ready-made operand
    w = torch.randn(128, in_dim, device="cuda", generator=g)
    want = ops.perturbed_linear(out, w, n_pop=batch, bm=1, t_steps=T, perturb=False, algo=ops.ALGO_TENSOR)
    ga = _lib.LinearArgs()
    res = torch.empty_like(want)
    ga.x, ga.t_steps, ga.n_pop, ga.bm, ga.k, ga.x_row_stride = out.data_ptr(), T, batch, 1, in_dim, in_dim
    ga.param, ga.a, ga.param_row_stride = w.data_ptr(), 128, in_dim
    ga.out, ga.out_row_stride, ga.out_scale, ga.algo = res.data_ptr(), 128, 1.0, ops.ALGO_TENSOR
    ga.x_half = half.data_ptr()
    need = int(L.hses_perturbed_linear_workspace_bytes(C.byref(ga)))
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    ga.workspace, ga.workspace_bytes = ws.data_ptr(), need
    ctx.profile_enable(False)
    assert L.hses_perturbed_linear(ctx.handle, stream, C.byref(ga)) == 0, L.hses_last_error()
    assert "split_x" not in {k for k, v in ctx.profile_read().items() if v[0]}
    assert torch.equal(res, want)
