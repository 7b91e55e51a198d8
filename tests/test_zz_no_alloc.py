"""The allocation-free update entry point, called through the C ABI.

Some callers of the library cannot allocate device memory (they live inside
another runtime's pool, or must not disturb the allocator mid-step), so
`hses_es_update_static` keeps its scratch in a fixed array inside the library
image.  It must give the same gradient as `hses_es_update`, call after call,
and must refuse shapes that do not fit its array.  This file sorts last so
that a run stopping at the first failure has already covered everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

KEY = 0xDAA66D2C7DDF743F


def _static(L, ctx, fitness, a, b, rank, sigma, first=0, n_total=None, epoch=0, reuse=0):
    n = fitness.numel()
    grad = torch.full((a, b), float("nan"), dtype=torch.float32, device=fitness.device)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.hses_es_update_static(ctx.handle, stream, C.c_uint64(KEY), epoch, reuse, first, n,
                                 n if n_total is None else n_total, rank, a, b, sigma,
                                 C.c_void_p(fitness.data_ptr()), C.c_void_p(grad.data_ptr()))
    return rc, grad


@pytest.mark.parametrize("a,b,rank,n", [(128, 784, 4, 256), (10, 128, 16, 64), (130, 70, 3, 18), (256, 512, 32, 512)])
def test_static_update_matches_workspace_update_twice(hs, a, b, rank, n):
    from hyperscalees_b200 import _lib, core, ops
    L = _lib.load()
    ctx = core.get_context(0)
    assert L.hses_es_update_static_scratch_bytes() == 16 << 20
    g = torch.Generator(device="cpu").manual_seed(a + n)
    for call in range(2):  # two calls in a row: the second one sees the first one's leftovers
        f = torch.randn(n, generator=g).cuda()
        want = ops.es_update(KEY, 3, 2, rank, a, b, 0.2, f, first_thread=4)
        rc, got = _static(L, ctx, f, a, b, rank, 0.2, first=4, epoch=3, reuse=2)
        assert rc == 0, L.hses_last_error()
        torch.cuda.synchronize()
        assert not torch.isnan(got).any()
        tol = 1e-3 * want.abs().max().item()
        assert (got - want).abs().max().item() <= tol


def test_static_update_matches_oracle(hs, oracle):
    from hyperscalees_b200 import _lib, core
    L = _lib.load()
    ctx = core.get_context(0)
    n, a, b, rank = 30, 24, 40, 8
    f = np.random.default_rng(1).standard_normal(n).astype(np.float32)
    rc, got = _static(L, ctx, torch.as_tensor(f, device="cuda"), a, b, rank, 0.3)
    assert rc == 0, L.hses_last_error()
    want = oracle.lora_grad(0.3, KEY, a, b, rank, f, [0] * n, list(range(n)), 0)
    assert np.abs(got.cpu().numpy() - want).max() <= 1e-3 * np.abs(want).max()


def test_static_update_leaves_device_memory_alone(hs, oracle):
    """A rank that no other call of this process has used: the entry point must not build (and
    allocate) a per-rank table on the way.  Free device memory as the driver reports it and the
    bytes torch's allocator holds are the same before and after."""
    from hyperscalees_b200 import _lib, core
    L = _lib.load()
    ctx = core.get_context(0)
    n, a, b, rank = 20, 33, 65, 7
    f = np.random.default_rng(5).standard_normal(n).astype(np.float32)
    fd = torch.as_tensor(f, device="cuda")
    _static(L, ctx, fd, 8, 8, 2, 0.1)          # the one-off address lookup of the array happens here
    grad = torch.empty((a, b), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    free0, reserved0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_reserved()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.hses_es_update_static(ctx.handle, stream, C.c_uint64(KEY), 0, 0, 0, n, n, rank, a, b, 0.3,
                                 C.c_void_p(fd.data_ptr()), C.c_void_p(grad.data_ptr()))
    assert rc == 0, L.hses_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0 and torch.cuda.memory_reserved() == reserved0
    want = oracle.lora_grad(0.3, KEY, a, b, rank, f, [0] * n, list(range(n)), 0)
    assert np.abs(grad.cpu().numpy() - want).max() <= 1e-3 * np.abs(want).max()


def test_static_update_rejects_what_does_not_fit(hs):
    from hyperscalees_b200 import _lib, core
    L = _lib.load()
    ctx = core.get_context(0)
    f = torch.zeros(4, device="cuda")
    rc, _ = _static(L, ctx, f, 4096, 4096, 16, 0.1)  # partial sums alone exceed the array
    assert rc == 1
    assert b"does not fit the built-in scratch" in L.hses_last_error()
    rc, _ = _static(L, ctx, torch.zeros(3, device="cuda"), 8, 8, 2, 0.1)  # odd member count
    assert rc == 1
