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
    (4, 64, 64, 16, 8, 1, 0),       # one 16-column item per tile (a per-head projection): the other columns of the
                                    # 128-wide MMA are zero rows of W and are never stored
    (4, 32, 256, 64, 8, 2, 2),      # a = 64: half a column tile, 16-column items
    (8, 32, 64, 96, 4, 1, 0),       # a = 96 with 32-column items (rank 4): three items per tile
    (8, 16, 96, 160, 16, 1, 0),     # two chunks of 128, the second one ragged
    (4, 64, 128, 320, 1, 1, 0),     # rank 1 (as rank 4), three chunks of 128, the last one half used
    (8, 16, 1024, 128, 16, 1, 0),   # the widest layer of the rows prepass: all 64 KB of a pair's B in shared memory
    (4, 32, 1000, 128, 8, 3, 1),    # k not a multiple of 128 there, three time steps, pairs cut at both ends
    (4, 32, 2048, 128, 4, 1, 0),    # rows longer than a warp's registers: the long-row prepass
    (4, 32, 1160, 128, 8, 2, 1),    # the same with rank 8, a ragged last piece, two time steps
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


@pytest.mark.parametrize("rank", [1, 2, 3])
@pytest.mark.parametrize("cached", [False, True])
@pytest.mark.parametrize("k", [192, 640, 1536])   # short rows, rows in registers, rows in pieces
def test_tensor_path_small_ranks(hs, oracle, rank, cached, k):
    """Ranks 1..3 run on the tensor-core path as rank 4 with zero columns: same stream positions
    (rank values per row), same results as the CPU restatement."""
    from hyperscalees_b200 import ops
    g = np.random.default_rng(rank)
    n_pop, bm, a, sigma = 6, 64, 256, 0.3
    x = g.standard_normal((n_pop, bm, k)).astype(np.float32)
    w = g.standard_normal((a, k)).astype(np.float32)
    cache = ops.FactorCache(KEY, 0, 0, rank, a, k, n_pairs=n_pop // 2, first_pair=1) if cached else None
    got = ops.perturbed_linear(torch.as_tensor(x, device="cuda"), torch.as_tensor(w, device="cuda"), n_pop=n_pop,
                               bm=bm, sigma=sigma, rank=rank, key=KEY, first_thread=2, algo=ops.ALGO_TENSOR,
                               cache=cache).cpu().numpy().reshape(n_pop, bm, a)
    for i in range(n_pop):
        want = oracle.do_mm(x[i], w, sigma, rank, KEY, (0, 2 + i), acc64=True)
        assert np.abs(got[i] - want).max() <= 2e-5 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("rank,perturb,k", [(1, True, 256), (16, True, 256), (4, False, 256), (1, True, 768),
                                               (1, True, 3072)])
def test_tensor_path_bf16_one_pass(hs, oracle, rank, perturb, k):
    """precision = BF16: x and the parameter rounded to bf16, one pass, fp32 accumulation; the
    rank-r term stays fp32.  Compared with the CPU product of the rounded operands plus the CPU
    rank-r term."""
    from hyperscalees_b200 import ops
    g = np.random.default_rng(10 + rank)
    n_pop, bm, a, sigma = 4, 64, 384, 0.2
    x = g.standard_normal((n_pop, bm, k)).astype(np.float32)
    w = (g.standard_normal((a, k)) * 0.02).astype(np.float32)
    rb = lambda v: torch.as_tensor(v).to(torch.bfloat16).to(torch.float32).numpy()
    got = ops.perturbed_linear(torch.as_tensor(x, device="cuda"), torch.as_tensor(w, device="cuda"), n_pop=n_pop,
                               bm=bm, sigma=sigma, rank=rank, key=KEY, perturb=perturb, algo=ops.ALGO_TENSOR,
                               precision=ops.PRECISION_BF16).cpu().numpy().reshape(n_pop, bm, a)
    for i in range(n_pop):
        want = oracle.do_mm(rb(x[i]), rb(w), sigma, rank, KEY, None, acc64=True)
        if perturb:
            want = want + (oracle.do_mm(x[i], w, sigma, rank, KEY, (0, i), acc64=True) -
                           oracle.do_mm(x[i], w, sigma, rank, KEY, None, acc64=True))
        assert np.abs(got[i] - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
    # the fp32-equivalent mode differs from it by the bf16 rounding of the operands, nothing like 2e-5
    full = ops.perturbed_linear(torch.as_tensor(x, device="cuda"), torch.as_tensor(w, device="cuda"), n_pop=n_pop,
                                bm=bm, sigma=sigma, rank=rank, key=KEY, perturb=perturb,
                                algo=ops.ALGO_TENSOR).cpu().numpy().reshape(n_pop, bm, a)
    assert np.abs(full - got).max() > 3e-5 * np.abs(full).max()   # (the rounding errors average out as k grows)


@pytest.mark.parametrize("algo_name,k,a,rank", [("TENSOR", 64, 256, 1), ("TENSOR", 192, 128, 4), ("SIMT", 96, 40, 1),
                                                ("SIMT", 64, 32, 3), ("TENSOR", 768, 128, 1), ("TENSOR", 512, 256, 8),
                                                ("TENSOR", 1280, 128, 8)])
def test_tmm_factor_order(hs, oracle, algo_name, k, a, rank):
    """do_Tmm (eggroll.rs:450-477): x @ param + (x·A)·Bᵀ for a parameter stored (in, out), whose
    factor block has the `out` rows first; the call takes the parameter transposed."""
    from hyperscalees_b200 import ops
    g = np.random.default_rng(k + a)
    n_pop, bm, sigma = 4, 64, 0.25
    x = g.standard_normal((n_pop, bm, k)).astype(np.float32)
    p_ref = g.standard_normal((k, a)).astype(np.float32)          # (in, out)
    got = ops.perturbed_linear(torch.as_tensor(x, device="cuda"), torch.as_tensor(p_ref.T.copy(), device="cuda"),
                               n_pop=n_pop, bm=bm, sigma=sigma, rank=rank, key=KEY, first_thread=6, tmm=True,
                               algo=getattr(ops, "ALGO_" + algo_name)).cpu().numpy().reshape(n_pop, bm, a)
    bs = float(np.float32(sigma) / np.sqrt(np.float32(rank)))
    for i in range(n_pop):
        A, B = oracle.lora_params(bs, KEY, rank, 0, 6 + i, k, a, 0)      # A (in, r) scaled, B (out, r)
        want = x[i].astype(np.float64) @ p_ref.astype(np.float64) + (x[i].astype(np.float64) @ A.astype(np.float64)) @ B.astype(np.float64).T
        assert np.abs(got[i] - want).max() <= 2e-5 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("perturb,cached", [(False, False), (True, False), (True, True)])
def test_operand_split_of_x_is_reused_across_projections(hs, perturb, cached):
    """Several projections of one activation (the per-head Q/K/V of a block): with reuse_x_split the
    second call keeps the first call's fp16 split of x and returns the bits of a call that splits again."""
    from hyperscalees_b200 import ops, core
    g = np.random.default_rng(21)
    n_pop, bm, k, a, rank = 4, 64, 64, 16, 8
    x = dev(g.standard_normal((n_pop, bm, k)).astype(np.float32))
    w1 = dev((g.standard_normal((a, k)) / 8).astype(np.float32))
    w2 = dev((g.standard_normal((a, k)) / 8).astype(np.float32))
    kw = dict(n_pop=n_pop, bm=bm, perturb=perturb, algo=ops.ALGO_TENSOR)
    def call(w, key, **extra):
        k2 = dict(kw)
        if perturb:
            k2.update(sigma=0.3, rank=rank, key=key)
            if cached:
                k2["cache"] = ops.FactorCache(key, 0, 0, rank, a, k, n_pairs=n_pop // 2)
        return ops.perturbed_linear(x, w, **k2, **extra)
    want = call(w2, 7).clone()
    call(w1, 5)
    got = call(w2, 7, reuse_x_split=True)
    assert core.get_context(0).device_status() == 0
    assert torch.equal(got, want)


@pytest.mark.parametrize("G,hd,k,rank,bm", [(4, 16, 64, 8, 32), (3, 32, 96, 4, 64), (2, 64, 256, 16, 16),
                                            (2, 32, 640, 1, 32)])
def test_grouped_projections_equal_the_separate_calls(hs, G, hd, k, rank, bm):
    """n_groups: G parameters stacked along the rows, each with its own noise, in one call that reads x
    once.  Every column must come out as in the call that projects its parameter alone."""
    from hyperscalees_b200 import ops
    g = np.random.default_rng(G * 100 + hd)
    n_pop, first = 8, 2
    x = dev(g.standard_normal((n_pop, bm, k)).astype(np.float32))
    ws = [dev((g.standard_normal((hd, k)) / np.sqrt(k)).astype(np.float32)) for _ in range(G)]
    keys = [KEY + 977 * j for j in range(G)]
    kw = dict(n_pop=n_pop, bm=bm, sigma=0.3, rank=rank, epoch=2, first_thread=first, noise_reuse=1)
    caches = [ops.FactorCache(keys[j], 2, 1, rank, hd, k, n_pop // 2, first_pair=first // 2) for j in range(G)]
    alone = [ops.perturbed_linear(x, ws[j], key=keys[j], cache=caches[j], algo=ops.ALGO_TENSOR, **kw) for j in range(G)]
    status_ok()
    grouped = ops.GroupedFactorCache(caches)
    got = ops.perturbed_linear(x, torch.cat(ws, 0), key=grouped.key, cache=grouped, n_groups=G, **kw)
    status_ok()
    want = torch.cat(alone, 1)
    scale = max(float(want.abs().max()), 1.0)
    assert float((got - want).abs().max()) <= 1e-6 * scale
    # a second projection of the same x keeps the operand split of the first
    again = ops.perturbed_linear(x, torch.cat(ws, 0), key=grouped.key, cache=grouped, n_groups=G, reuse_x_split=True, **kw)
    assert torch.equal(again, got)


def test_grouped_projections_refuse_what_they_do_not_cover(hs):
    from hyperscalees_b200 import ops, _lib
    x = torch.randn(8, 32, 64, device="cuda")
    ws = [torch.randn(16, 64, device="cuda") for _ in range(2)]
    caches = [ops.FactorCache(KEY + j, 0, 0, 4, 16, 64, 4) for j in range(2)]
    grouped = ops.GroupedFactorCache(caches)
    with pytest.raises(_lib.HsesError):   # 16-column groups need rank >= 8 (a ring item of rank 4 spans 32 columns)
        ops.perturbed_linear(x, torch.cat(ws, 0), n_pop=8, bm=32, sigma=0.1, rank=4, key=grouped.key, cache=grouped,
                             n_groups=2)


@pytest.mark.parametrize("extra", [dict(t_steps=2), dict(lif=True, tau_m=2.0, v_th=0.05), dict(precision=1)])
def test_grouped_projections_with_steps_lif_and_one_pass(hs, extra):
    """The grouped call in the other modes of the tensor-core path: several time steps, the fused LIF
    step, bf16 operands in one pass."""
    from hyperscalees_b200 import ops
    G, hd, k, rank, bm, n_pop, first = 2, 32, 128, 8, 32, 8, 0
    t_steps = extra.get("t_steps", 1)
    g = np.random.default_rng(5)
    x = dev(g.standard_normal((t_steps, n_pop, bm, k)).astype(np.float32))
    ws = [dev((g.standard_normal((hd, k)) / np.sqrt(k)).astype(np.float32)) for _ in range(G)]
    keys = [KEY + 31 * j for j in range(G)]
    kw = dict(n_pop=n_pop, bm=bm, sigma=0.3, rank=rank, epoch=0, first_thread=first, noise_reuse=0, **extra)
    caches = [ops.FactorCache(keys[j], 0, 0, rank, hd, k, n_pop // 2) for j in range(G)]
    alone = [ops.perturbed_linear(x, ws[j], key=keys[j], cache=caches[j], algo=ops.ALGO_TENSOR, **kw) for j in range(G)]
    grouped = ops.GroupedFactorCache(caches)
    got = ops.perturbed_linear(x, torch.cat(ws, 0), key=grouped.key, cache=grouped, n_groups=G, **kw)
    status_ok()
    want = torch.cat(alone, 1)
    if extra.get("lif"):
        assert float((got != want).float().mean()) <= 1e-4   # 0/1 spikes; a current on the threshold may flip
        assert 0.02 < float(want.mean()) < 0.98
    else:
        assert float((got - want).abs().max()) <= 1e-6 * max(float(want.abs().max()), 1.0)


@pytest.mark.parametrize("k,rank,precision,perturb", [(256, 8, 0, True), (640, 1, 1, True), (3072, 1, 1, True),
                                                      (1536, 4, 0, True), (256, 8, 0, False), (2304, 16, 0, True)])
def test_relu_square_on_the_input_equals_the_pass_of_its_own(hs, k, rank, precision, perturb):
    """x_op: the layer's input is relu(x)^2, applied where the prepass reads x (rows in registers, short or
    in pieces), or — clean calls, shapes whose prepass is the block kernel — by one pass before the call."""
    from hyperscalees_b200 import ops
    g = np.random.default_rng(k + rank)
    n_pop, bm, a = 8, 32, 128
    x = dev(g.standard_normal((n_pop, bm, k)).astype(np.float32))
    w = dev((g.standard_normal((a, k)) / np.sqrt(k)).astype(np.float32))
    kw = dict(n_pop=n_pop, bm=bm, sigma=0.3, rank=rank, key=KEY, precision=precision, perturb=perturb)
    want = ops.perturbed_linear(ops.relu_square(x), w, **kw)
    got = ops.perturbed_linear(x, w, x_relu_square=True, **kw)
    status_ok()
    assert torch.equal(got, want)
