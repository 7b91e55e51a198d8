"""Chunked accumulation of the update (accumulated_update / accumulated_update_cached,
eggroll.rs:550-702) against the one-shot do_updates — the equivalence the reference asserts in
eggroll.rs:1297-1369 (K chunks == full batch, solver step counter advances once) and that the
trainer's --verify mode re-checks (accumulate_train.rs:381-559)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(solver):
    from hyperscalees_b200 import noiser
    g = torch.Generator(device="cuda").manual_seed(11)
    params = [torch.randn(24, 40, device="cuda", generator=g), torch.randn(10, 24, device="cuda", generator=g),
              torch.ones(1, 1, device="cuda")]
    es = [noiser.MM_PARAM, noiser.MM_PARAM, noiser.PARAM]
    keys = [(i + 1) * 0x9E3779B97F4A7C15 % (1 << 64) for i in range(3)]
    frozen, nz = noiser.init_noiser(params, 0.3, 0.05, 0, False, 0, 4, solver)
    return params, es, keys, frozen, nz


@pytest.mark.parametrize("solver_name", ["sgd", "adamw"])
def test_four_update_paths_agree(solver_name):
    from hyperscalees_b200 import noiser
    mk = (lambda: noiser.Solver.sgd(0.05)) if solver_name == "sgd" else (lambda: noiser.Solver.adamw(0.05))
    batch, accumulate = 96, 4
    chunk = batch // accumulate
    raw = torch.randn(batch, device="cuda", generator=torch.Generator(device="cuda").manual_seed(2))
    tids = list(range(batch))
    infos = [noiser.IterInfo(3, t) for t in tids]

    outs = []
    # 1: one-shot update of the whole batch
    params, es, keys, frozen, nz = _setup(mk())
    conv = noiser.EggRoll().convert_fitnesses(frozen, nz, raw)
    outs.append(noiser.EggRoll().do_updates(frozen, nz, params, keys, conv, infos, es))
    assert nz.opt_state.step == (0 if solver_name == "sgd" else 1)
    # 2: K chunks, factors regenerated per chunk
    params, es, keys, frozen, nz = _setup(mk())
    outs.append(noiser.accumulated_update(frozen, nz, params, keys, es, conv, tids, 3, accumulate, chunk))
    assert nz.opt_state.step == (0 if solver_name == "sgd" else 1)   # once, not K times
    # 3: K chunks reading the noise cache
    params, es, keys, frozen, nz = _setup(mk())
    cache = noiser.build_lora_noise_cache(params, keys, es, batch, frozen.rank, frozen.noise_reuse, epoch=3)
    assert cache.buffers[2] is None and cache.buffers[0] is not None
    outs.append(noiser.accumulated_update_cached(frozen, nz, params, keys, es, conv, tids, 3, accumulate,
                                                 chunk, cache))
    # 4: a single chunk through the accumulating path
    params, es, keys, frozen, nz = _setup(mk())
    outs.append(noiser.accumulated_update(frozen, nz, params, keys, es, conv, tids, 3, 1, batch))

    ref = outs[0]
    for other in outs[1:]:
        for p0, want, got in zip(params, ref, other):
            moved = (want - p0).abs().max().item()
            assert moved > 0
            assert (got - want).abs().max().item() <= 1e-3 * moved + 1e-6
    # cached and uncached chunking read the same factors: identical bits
    for a, b in zip(outs[1], outs[2]):
        assert torch.equal(a, b)


def test_accumulated_update_rejects_broken_pairs():
    from hyperscalees_b200 import noiser
    params, es, keys, frozen, nz = _setup(noiser.Solver.sgd(0.1))
    conv = torch.zeros(6, device="cuda")
    with pytest.raises(ValueError):
        noiser.accumulated_update(frozen, nz, params, keys, es, conv, [0, 1, 2, 3, 4, 5], 0, 2, 3)
    with pytest.raises(ValueError):
        noiser.accumulated_update(frozen, nz, params, keys, es, conv, [1, 2, 3, 4, 5, 6], 0, 3, 2)
