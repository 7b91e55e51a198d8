"""RWKV-7 TimeMixing.forward (hyperscalees-models/src/llm.rs:348-479) assembled from the library's
kernels against a numpy composition of the CPU restatement's pieces (token shift, WKV-7
recurrence, group norm) on the same seeded inputs."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

VEC = ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g", "w0", "v0", "a0", "k_k", "k_a")


def make_weights(g, C, H, S, kdim):
    f = lambda *s, sc=1.0: (g.standard_normal(s) * sc).astype(np.float32)
    w = {n: f(C, sc=0.3) for n in VEC}
    w["x_r"], w["x_w"], w["x_k"], w["x_v"], w["x_a"], w["x_g"] = (g.random(C).astype(np.float32) for _ in range(6))
    w["r_k"] = f(H, S, sc=0.3)
    for n in ("receptance", "key", "value", "output"):
        w[n] = f(C, C, sc=1.0 / np.sqrt(C))
    for n in ("w1", "v1", "a1", "g1"):
        w[n] = f(C, kdim, sc=1.0 / np.sqrt(C))
    for n in ("w2", "v2", "a2", "g2"):
        w[n] = f(kdim, C, sc=1.0 / np.sqrt(kdim))
    w["ln_x_weight"] = (1.0 + f(C, sc=0.1)).astype(np.float32)
    w["ln_x_bias"] = f(C, sc=0.1)
    return w


def oracle_forward(oracle, w, x, state, v_first, length, ns, H, S, layer_id):
    f32 = np.float32
    T, C = x.shape
    sig = lambda z: (f32(1.0) / (f32(1.0) + np.exp(-z))).astype(f32)
    mix = lambda n: oracle.token_shift_mix(x, state[0], w[n], ns)
    xr, xw, xk, xv, xa, xg = (mix(n) for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g"))
    lin = lambda n, z: (z @ w[n].T).astype(f32)
    tmm = lambda n, z: (z @ w[n]).astype(f32)
    r = lin("receptance", xr)
    inner_w = w["w0"][None] + tmm("w2", np.tanh(tmm("w1", xw)))
    wdec = (-np.logaddexp(f32(0.0), -inner_w) - f32(0.5)).astype(f32)
    k = lin("key", xk)
    v = lin("value", xv)
    if layer_id == 0:
        v_first = v.copy()
    else:
        v = v + (v_first - v) * sig(w["v0"][None] + tmm("v2", np.tanh(tmm("v1", xv))))
    a = sig(w["a0"][None] + tmm("a2", np.tanh(tmm("a1", xa))))
    gte = tmm("g2", sig(tmm("g1", xg)))
    kk3 = (k * w["k_k"][None]).reshape(T, H, S)
    kk = (kk3 / np.maximum(np.sqrt((kk3 ** 2).sum(axis=2, keepdims=True)), 1e-12)).reshape(T, C).astype(f32)
    k = (k * (w["k_a"][None] * (a - f32(1.0)) + f32(1.0))).astype(f32)
    new_state = state.copy()
    new_state[0] = x[length - 1]
    s0 = state[1:1 + S].reshape(H, S, S)
    sh = lambda z: np.ascontiguousarray(z.reshape(T, H, S).astype(f32))
    args = [sh(r), sh(wdec), sh(k), sh(v), sh(-kk), sh(kk * a)]
    nsu = ns.astype(np.uint8)
    if length >= T:
        s_keep, out = oracle.wkv7(*args, s0, nsu)
    else:
        s_keep, o1 = oracle.wkv7(*[z[:length] for z in args], s0, nsu[:length])
        _, o2 = oracle.wkv7(*[z[length:] for z in args], s_keep, nsu[length:])
        out = np.concatenate([o1, o2], axis=0)
    new_state[1:1 + S] = s_keep.reshape(S, C)
    y = oracle.group_norm(out.reshape(T, C), H, w["ln_x_weight"], w["ln_x_bias"], eps=64e-5)
    bonus = (r.reshape(T, H, S) * k.reshape(T, H, S) * w["r_k"].reshape(1, H, S)).sum(axis=2, keepdims=True)
    y = (y + (bonus * v.reshape(T, H, S)).reshape(T, C)) * gte
    return lin("output", y.astype(f32)), new_state, v_first


@pytest.mark.parametrize("layer_id,length", [(0, 12), (1, 12), (1, 9)])
def test_time_mixing_matches_oracle_composition(hs, oracle, layer_id, length):
    from hyperscalees_b200.models import TimeMixing
    g = np.random.default_rng(31 + layer_id)
    T, H, S, kdim = 12, 2, 32, 8
    C = H * S
    w = make_weights(g, C, H, S, kdim)
    x = g.standard_normal((T, C)).astype(np.float32)
    state = (g.standard_normal((1 + S, C)) * 0.1).astype(np.float32)
    v_first = g.standard_normal((T, C)).astype(np.float32)
    ns = np.zeros(T, bool)
    ns[5] = True
    dev = lambda z: torch.as_tensor(z, device="cuda")
    tm = TimeMixing({n: dev(z) for n, z in w.items()})
    out, st, vf = tm.forward(dev(x), dev(state), dev(v_first), length, dev(ns), H, S, layer_id)
    wo, ws, wv = oracle_forward(oracle, w, x, state, v_first, length, ns, H, S, layer_id)
    tol = lambda z: 2e-4 * max(1.0, np.abs(z).max())
    assert np.abs(out.cpu().numpy() - wo).max() <= tol(wo)
    assert np.abs(st.cpu().numpy() - ws).max() <= tol(ws)
    assert np.abs(vf.cpu().numpy() - wv).max() <= tol(wv)
    assert np.array_equal(st[0].cpu().numpy(), x[length - 1])


def test_time_mixing_noise_changes_output_and_antithetic_pairs_differ(hs):
    from hyperscalees_b200.models import TimeMixing, default_base_keys
    from hyperscalees_b200 import noiser
    g = np.random.default_rng(5)
    T, H, S, kdim = 6, 2, 32, 8
    C = H * S
    w = {n: torch.as_tensor(z, device="cuda") for n, z in make_weights(g, C, H, S, kdim).items()}
    tm = TimeMixing(w)
    mats = [n for n in w if w[n].dim() == 2 and n != "r_k"]
    keys = dict(zip(mats, default_base_keys(len(mats))))
    frozen, params = noiser.init_noiser([w[n] for n in mats], 0.05, 0.01, 0, False, 0, 4, noiser.Solver.sgd(0.01))
    nz = noiser.EggRoll()
    x = torch.as_tensor(g.standard_normal((T, C)).astype(np.float32), device="cuda")
    state = torch.zeros(1 + S, C, device="cuda")
    vf = torch.zeros(T, C, device="cuda")
    run = lambda info: tm.forward(x, state, vf, T, None, H, S, 0,
                                  noise=None if info is None else (nz, frozen, params, keys, info))[0]
    clean, plus, minus = run(None), run(noiser.IterInfo(0, 0)), run(noiser.IterInfo(0, 1))
    assert (plus - clean).abs().max() > 1e-4 and (minus - clean).abs().max() > 1e-4
    assert (plus - minus).abs().max() > 1e-4
