"""Explicit-input paired einsum (oxide seam `einsum_pair_fused`) against an f64 host
reference on the fixture generator and shape list of the reference's own kernel check
(hyperscalees-kernels/src/einsum_pair_fused_oxide.rs:425-467, 760-795); pass criterion
of that check: |got - exp| <= 1e-4 * (1 + |exp|)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

M64 = (1 << 64) - 1


LCG_A, LCG_C = 6364136223846793005, 1442695040888963407


def lcg_fill(seed: int, n: int):
    """Uniform values in [-1, 1) from the 64-bit LCG the reference check uses; returns
    (values, next seed).  State i is P[i]*seed + Q[i] (mod 2^64); P and Q are built by doubling
    (state i+k = P[i]*state k + Q[i]), so the stream costs a few numpy passes instead of a Python loop."""
    P = np.empty(n + 1, dtype=np.uint64)
    Q = np.empty(n + 1, dtype=np.uint64)
    P[0], Q[0] = 1, 0
    pk, qk, k = LCG_A, LCG_C, 1          # P and Q of index k
    with np.errstate(over="ignore"):
        while k <= n:
            m = min(k, n + 1 - k)
            P[k:k + m] = P[:m] * np.uint64(pk)
            Q[k:k + m] = P[:m] * np.uint64(qk) + Q[:m]
            pk, qk, k = (pk * pk) & M64, (pk * qk + qk) & M64, 2 * k
        state = P[1:] * np.uint64(seed) + Q[1:]
    out = (((state >> np.uint64(33)) & np.uint64(0xFFFFFFFF)).astype(np.float64) / float(1 << 31) - 1.0).astype(np.float32)
    return out, (int(state[-1]) if n else seed)


def host_reference(a_t, b_t, scores):
    half, r, a = a_t.shape
    f = (scores[:half] + scores[half:]).astype(np.float64)   # the kernel's f32 sum is within 2^-24 of this
    a64 = a_t.astype(np.float64).reshape(half * r, a)
    b64 = b_t.astype(np.float64).reshape(half * r, -1)
    g_raw = (a64 * np.repeat(f, r)[:, None]).T @ b64
    g_ones = 2.0 * (a64.T @ b64)
    return g_raw, g_ones


SHAPES = [  # (half, r, a, b, a_pitch, b_pitch); pitch 0 = dense
    (8, 3, 2, 3, 0, 0), (2, 16, 8, 8, 0, 0), (5, 4, 10, 17, 0, 0), (64, 16, 32, 48, 0, 0),
    (200, 64, 128, 784, 0, 0), (1000, 16, 32, 48, 0, 0), (1000, 16, 32, 48, 32 + 32, 64),
    (33, 7, 130, 65, 136, 72), (1, 1, 1, 1, 0, 0),
    # long contractions over 16-byte aligned rows: the tensor-core kernel (whole pairs per 64-row
    # k-block for r = 4, 16; one pair per block for r = 64; a zero-filled second block for r = 96; a
    # zero-filled tail for r = 48; ragged output tiles; a pair count that does not fill the last block)
    (8203, 4, 64, 64, 0, 0), (400, 96, 130, 68, 136, 72), (700, 48, 200, 100, 0, 0), (600, 64, 256, 784, 0, 0),
    (4100, 8, 40, 300, 0, 0),
    # the same length with rows that are not 16-byte multiples: fp32 kernel
    (2100, 16, 33, 47, 0, 0),
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
    # Contractions of 32768 rows and more over 16-byte aligned rows run on the tensor cores, whose
    # accumulator adds with truncation (a relative 2^-24 or so per MMA, towards zero, over chains of
    # 192 MMAs): those are held to 3e-5 of the output's largest magnitude (the update's stated
    # tolerance is 1e-3 relative); everything else, the reference's own shape list included, to the
    # reference check's criterion.
    tensor = half * r >= 32768 and ap % 4 == 0 and bp % 4 == 0
    for got, exp in ((g_raw, exp_raw), (g_ones, exp_ones)):
        got = got.cpu().numpy().astype(np.float64)
        assert got.shape == (a, b)
        if tensor:
            assert np.abs(got - exp).max() <= 3e-5 * np.abs(exp).max()
        else:
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


def test_einsum_pair_operand_ranges():
    """The tensor-core kernel scales each operand by a power of two found from its largest magnitude:
    operands far from 1 (1e5, 1e-7, scores of 1e3) must come out with the same relative accuracy."""
    from hyperscalees_b200 import kernels
    half, r, a, b = 2100, 16, 96, 160
    rng = np.random.default_rng(11)
    av = (rng.uniform(-1, 1, (half, r, a)) * 1e5).astype(np.float32)
    bv = (rng.uniform(-1, 1, (half, r, b)) * 1e-7).astype(np.float32)
    sv = (rng.uniform(-1, 1, 2 * half) * 1e3).astype(np.float32)
    g_raw, g_ones = kernels.einsum_pair_fused(torch.from_numpy(av).cuda(), torch.from_numpy(bv).cuda(),
                                              torch.from_numpy(sv).cuda())
    exp_raw, exp_ones = host_reference(av, bv, sv)
    for got, exp in ((g_raw, exp_raw), (g_ones, exp_ones)):
        got = got.cpu().numpy().astype(np.float64)
        assert np.all(np.isfinite(got))
        assert np.abs(got - exp).max() <= 1e-5 * np.abs(exp).max()
    # all-zero operands: the ranges fall back to exponent 0, the sums are exact zeros
    z_raw, z_ones = kernels.einsum_pair_fused(torch.zeros(half, r, a, device="cuda"), torch.from_numpy(bv).cuda(),
                                              torch.from_numpy(sv).cuda())
    assert not z_raw.any() and not z_ones.any()
