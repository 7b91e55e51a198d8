"""The raw-kernel seam of the reference (hyperscalees/src/oxide.rs wrappers over
the hyperscalees-kernels crate), kept under the same names so a trainer that
called `oxide::lif_fused` / `oxide::poisson_encode_fused` finds them here."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import ops

N_VALUES_PER_THREAD = 128   # hyperscalees-kernels/src/lib.rs:19
VECTORS_PER_THREAD = 32     # hyperscalees-kernels/src/lib.rs:21


def lif_fused(cur: torch.Tensor, v0: Optional[torch.Tensor], tau_m: float, v_th: float) -> torch.Tensor:
    """oxide.rs:489-543: cur (T, n, h), v0 (n, h) -> spikes (T, n, h); v0 is not modified."""
    v = None if v0 is None else v0.detach().clone()
    return ops.lif_scan(cur, tau_m, v_th, v=v)


def poisson_encode_fused(images: torch.Tensor, t: int, seeds: Sequence[int]) -> torch.Tensor:
    """oxide.rs:573-625, with the four seed words passed in instead of being drawn
    from the wall clock (oxide.rs:205-223)."""
    if t > 8:
        raise ValueError("poisson_encode_fused: t must be <= 8 (oxide.rs:578-580)")
    return ops.poisson_encode(images, t, seeds)
