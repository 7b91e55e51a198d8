"""The host-side mirror of the noiser/models crates, exercised the way the
reference's own unit tests exercise the Rust functions."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def bits(t):
    return t.detach().cpu().numpy().view(np.uint32)


def test_get_lora_update_params_shapes_and_sign(hs, oracle):
    # hyperscalees-noiser/src/eggroll.rs:1075-1099
    from hyperscalees_b200 import noiser
    A0, B0 = noiser.get_lora_update_params(0.1, 42, 3, noiser.IterInfo(0, 0), 4, 5, 0)
    A1, B1 = noiser.get_lora_update_params(0.1, 42, 3, noiser.IterInfo(0, 1), 4, 5, 0)
    assert A0.shape == (4, 3) and B0.shape == (5, 3)
    assert torch.equal(B0, B1) and torch.equal(A0, -A1)
    wa, wb = oracle.lora_params(0.1, 42, 3, 0, 0, 4, 5, 0)
    assert np.array_equal(bits(A0), wa.view(np.uint32)) and np.array_equal(bits(B0), wb.view(np.uint32))


def test_batched_lora_noise_matches_per_thread(hs):
    # eggroll.rs:1101-1129: bit-equality between the batched and the per-member form
    from hyperscalees_b200 import noiser
    tids = [0, 1, 5, 8, 13]
    A, B = noiser.batched_lora_noise(0.05, 1234, 4, tids, 3, 2, 6, 9)
    for i, tid in enumerate(tids):
        a1, b1 = noiser.get_lora_update_params(0.05, 1234, 4, noiser.IterInfo(3, tid), 6, 9, 2)
        assert torch.equal(A[i], a1) and torch.equal(B[i], b1)


def test_deterministic_noise_repeatable_and_continuing(hs, oracle):
    # noiser.rs:686-700
    from hyperscalees_b200 import noiser
    r1 = noiser.DeterministicNoise(77)
    x = r1.normal_tensor([3, 4])
    y = r1.normal_tensor([5])
    want = oracle.normals(77, 17)
    assert np.array_equal(bits(x).reshape(-1), want[:12].view(np.uint32))
    assert np.array_equal(bits(y), want[12:].view(np.uint32))
    assert torch.equal(noiser.DeterministicNoise(77).normal_tensor([3, 4]), x)


def test_do_mm_none_is_clean_and_member_matches_oracle(hs, oracle):
    from hyperscalees_b200 import noiser
    g = np.random.default_rng(2)
    x = g.standard_normal((5, 12)).astype(np.float32)
    w = g.standard_normal((7, 12)).astype(np.float32)
    frozen, nz = noiser.init_noiser([], 0.4, 0.1, 0, False, 0, 2, noiser.Solver.sgd(0.1))
    dx, dw = torch.as_tensor(x, device="cuda"), torch.as_tensor(w, device="cuda")
    er = noiser.EggRoll()
    clean = er.do_mm(frozen, nz, dw, 11, None, dx).cpu().numpy()
    assert np.allclose(clean, x @ w.T, atol=1e-5)
    noisy = er.do_mm(frozen, nz, dw, 11, noiser.IterInfo(0, 3), dx).cpu().numpy()
    assert np.allclose(noisy, oracle.do_mm(x, w, 0.4, 2, 11, (0, 3), 0), atol=1e-5)
    # do_Tmm: x @ param + x A B^T (eggroll.rs:450-477)
    xt = g.standard_normal((5, 7)).astype(np.float32)
    A, B = oracle.lora_params(np.float32(0.4) / np.sqrt(np.float32(2)), 11, 2, 0, 3, 7, 12, 0)
    want = xt @ w + (xt @ A) @ B.T
    got = er.do_Tmm(frozen, nz, dw, 11, noiser.IterInfo(0, 3), torch.as_tensor(xt, device="cuda"))
    assert np.allclose(got.cpu().numpy(), want, atol=1e-4)
    with pytest.raises(NotImplementedError):
        er.do_emb(frozen, nz, dw, 11, None, None)


def test_get_noisy_standard(hs, oracle):
    from hyperscalees_b200 import noiser
    p = torch.ones(2, 3, device="cuda")
    frozen, nz = noiser.init_noiser([p], 0.3, 0.1, 0, False, 0, 1, noiser.Solver.sgd(0.1))
    er = noiser.EggRoll()
    assert torch.equal(er.get_noisy_standard(frozen, nz, p, 5, None), p)
    got = er.get_noisy_standard(frozen, nz, p, 5, noiser.IterInfo(0, 1)).cpu().numpy()
    assert np.allclose(got, 1.0 + oracle.nonlora_params(0.3, 5, 0, 1, 2, 3, 0), atol=1e-6)
    frozen.freeze_nonlora = True
    assert torch.equal(er.get_noisy_standard(frozen, nz, p, 5, noiser.IterInfo(0, 1)), p)


def test_do_updates_sgd_full_pipeline(hs, oracle):
    # eggroll.rs:1234-1272: two envs, dense update, shape [1, 2], lr=0.1, sigma=0.5
    from hyperscalees_b200 import noiser
    lr, sigma, key = 0.1, 0.5, 99
    frozen, nz = noiser.init_noiser([], sigma, lr, 0, False, 0, 1, noiser.Solver.sgd(lr))
    p = torch.tensor([[1.0, -1.0]], device="cuda")
    fit = torch.tensor([1.0, 2.0], device="cuda")
    infos = [noiser.IterInfo(0, 0), noiser.IterInfo(0, 1)]
    g = np.zeros(2, np.float32)
    for i, info in enumerate(infos):
        te, tt, sign = noiser.epoch_thread_sign(info, 0)
        g += np.float32([1.0, 2.0][i]) * np.float32(sign) * np.float32(sigma) * oracle.normals(oracle.noise_seed(key, te, tt), 2)
    expected = np.array([1.0, -1.0], np.float32) + lr * (g / 2) * np.sqrt(2.0)
    out = noiser.EggRoll().do_updates(frozen, nz, [p], [key], fit, infos, [noiser.PARAM])
    assert np.allclose(out[0].cpu().numpy().reshape(-1), expected, atol=1e-4)
    assert torch.equal(p, torch.tensor([[1.0, -1.0]], device="cuda"))  # inputs untouched


def test_do_updates_single_member_and_scattered_ids(hs, oracle):
    # eggroll.rs:1173-1204 uses N = 1; arbitrary thread ids must work as well
    from hyperscalees_b200 import noiser
    frozen, nz = noiser.init_noiser([], 0.5, 0.1, 0, False, 0, 1, noiser.Solver.sgd(0.1))
    er = noiser.EggRoll()
    p = torch.zeros(2, 2, device="cuda")
    g1 = er.grads(frozen, nz, [p], [7], torch.tensor([1.0], device="cuda"), [noiser.IterInfo(0, 0)], [noiser.MM_PARAM])
    want = oracle.lora_grad(0.5, 7, 2, 2, 1, [1.0], [0], [0])
    assert np.allclose(g1[0].cpu().numpy(), want, atol=1e-5)
    infos = [noiser.IterInfo(0, 5), noiser.IterInfo(0, 2), noiser.IterInfo(0, 9)]
    f = [0.3, -1.0, 2.0]
    g2 = er.grads(frozen, nz, [p], [7], torch.tensor(f, device="cuda"), infos, [noiser.MM_PARAM])
    want = oracle.lora_grad(0.5, 7, 2, 2, 1, f, [0, 0, 0], [5, 2, 9])
    assert np.allclose(g2[0].cpu().numpy(), want, atol=1e-5)


def test_noop_and_frozen_classes_give_zero_grad(hs):
    from hyperscalees_b200 import noiser
    frozen, nz = noiser.init_noiser([], 0.5, 0.1, 0, True, 0, 1, noiser.Solver.sgd(0.1))
    p = torch.ones(2, 2, device="cuda")
    f = torch.tensor([1.0, -1.0], device="cuda")
    infos = [noiser.IterInfo(0, 0), noiser.IterInfo(0, 1)]
    out = noiser.EggRoll().do_updates(frozen, nz, [p, p], [1, 2], f, infos, [noiser.PARAM, noiser.EXCLUDED])
    assert torch.equal(out[0], p) and torch.equal(out[1], p)


def test_adam_step_counter_and_trust_region(hs, oracle):
    from hyperscalees_b200 import noiser
    p = torch.randn(3, 4, device="cuda")
    g = torch.randn(3, 4, device="cuda") * 10
    s = noiser.Solver.trust_region(1.0, noiser.Solver.adam(0.01))
    st = s.init_state([p])
    out = s.update([p], [g], st)
    assert st.step == 1
    scale = oracle.clip_scale([g.cpu().numpy()], 1.0)
    want, _, _ = oracle.solver_update(oracle.ADAM, 1, p.cpu().numpy(), g.cpu().numpy() * np.float32(scale), lr=0.01)
    assert np.allclose(out[0].cpu().numpy(), want, atol=1e-5)


def test_eggroll_bs_noiser(hs, oracle):
    """EggRollBS (eggroll_bs.rs): masked members are clean, per-direction fitness, trust-region solver."""
    from hyperscalees_b200 import noiser, ops
    bs = noiser.EggRollBS()
    p = torch.randn(6, 8, device="cuda")
    frozen, nz = bs.init_noiser([p], 0.5, 0.1, 4, False, 0, 2, 1.0, noiser.Solver.sgd(0.1))
    assert frozen.solver.kind == "trust_region" and frozen.group_size == 4
    x = torch.randn(3, 8, device="cuda")
    clean = bs.do_mm(frozen, nz, p, 9, None, x)
    # eggroll_bs.rs:430-464: directions 0 and 1 of every group are silenced, the others are not
    for tid, masked in ((0, True), (1, True), (2, False), (5, True), (6, False), (7, False)):
        y = bs.do_mm(frozen, nz, p, 9, noiser.IterInfo(0, tid), x)
        assert torch.equal(y, clean) == masked
        plain = noiser.EggRoll().do_mm(frozen, nz, p, 9, noiser.IterInfo(0, tid), x)
        if not masked:
            assert torch.equal(y, plain)
    # per-direction fitness against the oracle
    raw = torch.randn(12 * 4, device="cuda") * 2 + 1
    got = bs.convert_fitnesses(frozen, nz, raw).cpu().numpy()
    want = oracle.convert_fitnesses_bs(raw.cpu().numpy(), 4)
    assert got.shape == (4,) and got[0] == 0.0 and got[1] == 0.0
    assert np.allclose(got, want, rtol=1e-5, atol=1e-6)
    # update: masked members contribute nothing
    fit = torch.tensor([3.0, -2.0, 1.0, 0.5], device="cuda")
    infos = [noiser.IterInfo(0, t) for t in range(4)]
    (g_bs,) = bs.grads(frozen, nz, [p], [9], fit, infos, [noiser.MM_PARAM])
    fit_masked = torch.tensor([0.0, 0.0, 1.0, 0.5], device="cuda")
    (g_ref,) = noiser.EggRoll().grads(frozen, nz, [p], [9], fit_masked, infos, [noiser.MM_PARAM])
    assert torch.equal(g_bs, g_ref)
    # eggroll_bs.rs:508-530: the combined gradient is clipped to the trust-region norm
    new = bs.do_updates(frozen, nz, [p], [9], fit * 100, infos, [noiser.MM_PARAM])
    step = (p - new[0]) / 0.1
    assert abs(float(step.norm()) - 1.0) <= 1e-3
