"""Explicit-input paired einsum (oxide seam `einsum_pair_fused`) against an f64 host
reference on the fixture generator and shape list of the reference's own kernel check
(hyperscalees-kernels/src/einsum_pair_fused_oxide.rs:425-467, 760-795); pass criterion
of that check: |got - exp| <= 1e-4 * (1 + |exp|)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

M64 = (1 << 64) - 1


def lcg_fill(seed: int, n: int):
    """Uniform values in [-1, 1) from the 64-bit LCG the reference check uses; returns
    (values, next seed)."""
    out = np.empty(n, dtype=np.float32)
    for i in range(n):
        seed = (seed * 6364136223846793005 + 1442695040888963407) & M64
        out[i] = np.float32(((seed >> 33) & 0xFFFFFFFF) / float(1 << 31) - 1.0)
    return out, seed


def host_reference(a_t, b_t, scores):
    half = a_t.shape[0]
    f = (scores[:half] + scores[half:]).astype(np.float64)
    a64, b64 = a_t.astype(np.float64), b_t.astype(np.float64)
    g_raw = np.einsum("i,ijm,ijn->mn", f, a64, b64)
    g_ones = 2.0 * np.einsum("ijm,ijn->mn", a64, b64)
    return g_raw, g_ones


SHAPES = [  # (half, r, a, b, a_pitch, b_pitch); pitch 0 = dense
    (8, 3, 2, 3, 0, 0), (2, 16, 8, 8, 0, 0), (5, 4, 10, 17, 0, 0), (64, 16, 32, 48, 0, 0),
    (200, 64, 128, 784, 0, 0), (1000, 16, 32, 48, 0, 0), (1000, 16, 32, 48, 32 + 32, 64),
    (33, 7, 130, 65, 136, 72), (1, 1, 1, 1, 0, 0),
]


@pytest.mark.parametrize("half,r,a,b,ap,bp", SHAPES)
def test_einsum_pair_matches_f64(half, r, a, b, ap, bp):
    from hyperscalees_b200 import kernels
    ap, bp = ap or a, bp or b
    seed = 0x9E3779B97F4A7C15 ^ (half * 1315423911 + r * 2654435761 + a * 97 + b)
    av, seed = lcg_fill(seed, half * r * ap)
    bv, seed = lcg_fill(seed, half * r * bp)
    sv, seed = lcg_fill(seed, 2 * half)
    a_full = torch.from_numpy(av.reshape(half, r, ap)).cuda()
    b_full = torch.from_numpy(bv.reshape(half, r, bp)).cuda()
    a_t, b_t = a_full[:, :, :a], b_full[:, :, :b]
    scores = torch.from_numpy(sv).cuda()
    g_raw, g_ones = kernels.einsum_pair_fused(a_t, b_t, scores)
    exp_raw, exp_ones = host_reference(av.reshape(half, r, ap)[:, :, :a], bv.reshape(half, r, bp)[:, :, :b], sv)
    for got, exp in ((g_raw, exp_raw), (g_ones, exp_ones)):
        got = got.cpu().numpy().astype(np.float64)
        assert got.shape == (a, b)
        assert np.all(np.abs(got - exp) <= 1e-4 * (1 + np.abs(exp)))
    # deterministic: the split-K partial sums are merged in a fixed order
    g2, o2 = kernels.einsum_pair_fused(a_t, b_t, scores)
    assert torch.equal(g2, g_raw) and torch.equal(o2, g_ones)


def test_einsum_pair_agrees_with_update_path():
    """The same contraction through the regenerating update entry point: build the factor
    cache of a layer, feed its A'/B' blocks and raw scores to einsum_pair, and compare
    with hses_es_update in raw-accumulate mode."""
    from hyperscalees_b200 import ops, kernels
    n, r, a, b = 256, 8, 48, 80
    key, epoch = 0x1234ABCD, 3
    cache = ops.FactorCache(key, epoch, 0, r, a, b, n // 2, device=torch.device("cuda"))
    a_t = cache.A.transpose(1, 2).contiguous()     # (half, r, a)
    b_t = cache.B.transpose(1, 2).contiguous()
    g = torch.Generator().manual_seed(5)
    scores = torch.randn(n, generator=g).cuda()
    g_raw, g_ones = kernels.einsum_pair_fused(a_t, b_t, scores)
    # pair member order of the population is (2i, 2i+1); einsum_pair pairs (i, i+half)
    inter = torch.empty_like(scores)
    inter[0::2], inter[1::2] = scores[: n // 2], -scores[n // 2:]
    ref = ops.es_update(key, epoch, 0, r, a, b, float(np.sqrt(r)), inter, mode=ops.UPDATE_RAW_ACC, cache=cache)
    assert torch.allclose(g_raw, ref, rtol=1e-4, atol=1e-4)


def test_einsum_pair_rejects_bad_shapes():
    from hyperscalees_b200 import kernels
    a_t = torch.zeros(4, 2, 8, device="cuda")
    b_t = torch.zeros(4, 3, 8, device="cuda")
    with pytest.raises(ValueError):
        kernels.einsum_pair_fused(a_t, b_t, torch.zeros(8, device="cuda"))
    with pytest.raises(ValueError):
        kernels.einsum_pair_fused(a_t, torch.zeros(4, 2, 8, device="cuda"), torch.zeros(7, device="cuda"))
