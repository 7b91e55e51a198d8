"""RWKV-7 language model over a population: the WKV-7 kernel against an independent golden case,
the stack against the CPU composition (oracle/rwkv_lm.py) member by member."""
import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def dev(a):
    return torch.as_tensor(np.ascontiguousarray(a), device="cuda")


def test_wkv7_kernel_against_the_golden_case(hs):
    """tests/golden/wkv7_golden.json: non-zero k, v, a, b and a mid-sequence restart (float64 values)."""
    from hyperscalees_b200 import ops
    d = json.load(open(os.path.join(HERE, "golden", "wkv7_golden.json")))
    I = {k: np.array(v, dtype=np.float32) for k, v in d["inputs"].items()}
    T, H, S = d["T"], d["H"], d["S"]
    # the kernel takes head sizes 32 and 64: embed the 4-wide case in the first components of a 32-wide head
    def wide(x, fill=0.0):
        out = np.full((1, T, H, 32), fill, np.float32)
        out[0, :, :, :S] = x
        return out
    st = np.zeros((1, H, 32, 32), np.float32)
    st[0, :, :S, :S] = I["state"]
    std = dev(st)
    out = ops.wkv7(dev(wide(I["r"])), dev(wide(I["w"])), dev(wide(I["k"])), dev(wide(I["v"])), dev(wide(I["a"])),
                   dev(wide(I["b"])), std, dev(I["new_starts"].astype(np.uint8).reshape(1, T))).cpu().numpy()
    want, want_s = np.array(d["out"]), np.array(d["state_out"])
    assert np.abs(out[0, :, :, :S] - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
    assert np.abs(out[0, :, :, S:]).max() == 0.0
    assert np.abs(std.cpu().numpy()[0, :, :S, :S] - want_s).max() <= 1e-5 * max(1.0, np.abs(want_s).max())


def np_model(m):
    cv = lambda t: t.cpu().numpy()
    layers = []
    for w in m.layers:
        layers.append({k: (tuple(cv(x) for x in v) if isinstance(v, tuple) else cv(v)) for k, v in w.items()})
    return {"emb": cv(m.emb), "head": cv(m.head)[:m.vocab], "head_padded": cv(m.head), "ln0": tuple(cv(x) for x in m.ln0),
            "ln_out": tuple(cv(x) for x in m.ln_out), "layers": layers, "keys": m.keys, "H": m.H, "S": m.S}


@pytest.mark.parametrize("perturb", [False, True])
def test_population_fitness_matches_the_cpu_composition(hs, oracle, perturb):
    from hyperscalees_b200.rwkv_lm import LmNoise, RwkvLM
    from oracle import rwkv_lm as RL
    n, T, vocab = 4, 32, 300
    m = RwkvLM(n_layer=2, d_model=128, vocab=vocab, head_size=64, lora_dims=(32, 32, 32, 128), seed=4, std=0.05)
    g = np.random.default_rng(4)
    ids = g.integers(0, vocab, (n, T)).astype(np.int32)
    noise = LmNoise(0.1, 1, first_thread=2) if perturb else None
    # four members of 32 tokens per pass: 128 rows, the smallest call the tensor-core product takes
    fit, logits = m.fitness(dev(ids), noise, chunk_members=4, head_members=4, want_logits=True)
    fit, logits = fit.cpu().numpy(), logits.cpu().numpy().reshape(n, T, vocab)
    npm = np_model(m)
    for j in range(n):
        nz = (0.1, 1, 0, 2 + j, 0) if perturb else None
        wf, wl = RL.member_fitness(npm, ids[j], nz, rows_in_call=n * T, head_rows_in_call=n * T)
        # an activation that lands on the other side of a bf16 rounding boundary moves one product
        # term by 2^-8 of itself: the logits are held to 1e-2, the token-averaged fitness to 1e-3
        assert np.abs(logits[j] - wl).max() <= 1e-2 * max(1.0, np.abs(wl).max())
        assert abs(fit[j] - wf) <= 1e-3 * max(1.0, abs(wf))
    if perturb:
        assert np.abs(logits[0] - logits[1]).max() > 0     # antithetic partners differ
    else:
        assert np.abs(fit - fit[0]).max() > 0              # different sequences, different fitness


@pytest.mark.parametrize("H,S,layer0", [(3, 64, True), (3, 64, False), (4, 32, False), (2, 128, False)])
def test_time_mixing_elementwise_kernels_against_the_composition(hs, H, S, layer0):
    """hses_rwkv_mix_prepare / hses_rwkv_mix_finish (llm.rs:396-440, 462-472) against the same formulas written
    out with array operations in fp64."""
    import torch
    from hyperscalees_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(H * S)
    rows, C = 37, H * S
    rnd = lambda *shape: torch.randn(*shape, device="cuda", generator=g)
    w_lin, v_raw, v_lin, v_first, a_lin, k_raw = (rnd(rows, C) * 2 for _ in range(6))
    w0, v0, a0, k_k, k_a = (rnd(C) for _ in range(5))
    got = ops.rwkv_mix_prepare(w_lin, v_raw, None if layer0 else v_lin, None if layer0 else v_first, a_lin, k_raw,
                               w0, None if layer0 else v0, a0, k_k, k_a, H)
    d = lambda t: t.double()
    sig = torch.sigmoid
    w_want = -torch.nn.functional.softplus(-(d(w0) + d(w_lin))) - 0.5
    v_want = d(v_raw) if layer0 else d(v_raw) + (d(v_first) - d(v_raw)) * sig(d(v0) + d(v_lin))
    a = sig(d(a0) + d(a_lin))
    kk3 = (d(k_raw) * d(k_k)).view(rows, H, S)
    kk = (kk3 / kk3.pow(2).sum(dim=2, keepdim=True).sqrt().clamp_min(1e-12)).reshape(rows, C)
    k_want = d(k_raw) * (d(k_a) * (a - 1.0) + 1.0)
    for name, gt, wt in zip(("w", "v", "k", "-kk", "kk*a"), got, (w_want, v_want, k_want, -kk, kk * a)):
        err = float((d(gt) - wt).abs().max())
        assert err <= 2e-6 * max(1.0, float(wt.abs().max())), (name, err)
    y_norm, r, gate, r_k = rnd(rows, C), rnd(rows, C), rnd(rows, C), rnd(H, S)
    out = ops.rwkv_mix_finish(y_norm, r, got[2], got[1], gate, r_k.reshape(-1), H)
    bonus = (d(r).view(rows, H, S) * d(got[2]).view(rows, H, S) * d(r_k).view(1, H, S)).sum(dim=2, keepdim=True)
    want = (d(y_norm) + (bonus * d(got[1]).view(rows, H, S)).reshape(rows, C)) * d(gate)
    assert float((d(out) - want).abs().max()) <= 1e-5 * max(1.0, float(want.abs().max()))


def test_token_shift_mix_of_several_coefficient_vectors(hs):
    """hses_token_shift_mix_multi gives what one hses_token_shift_mix call per coefficient vector gives."""
    import torch
    from hyperscalees_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(11)
    T, c = 50, 96
    x = torch.randn(T, c, device="cuda", generator=g)
    state = torch.randn(c, device="cuda", generator=g)
    ns = torch.zeros(T, dtype=torch.uint8, device="cuda")
    ns[[0, 17, 33]] = 1
    coefs = [torch.rand(c, device="cuda", generator=g) for _ in range(6)]
    got = ops.token_shift_mix_multi(x, state, coefs, ns)
    for cf, o in zip(coefs, got):
        assert torch.equal(o, ops.token_shift_mix(x, state, cf, ns))
