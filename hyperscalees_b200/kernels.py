"""The raw-kernel seam of the reference (hyperscalees/src/oxide.rs wrappers over
the hyperscalees-kernels crate), kept under the same names so a trainer that
called `oxide::lif_fused` / `oxide::poisson_encode_fused` finds them here."""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

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


def einsum_pair_fused(a_t: torch.Tensor, b_t: torch.Tensor,
                      scores: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """oxide.rs:325-462: a_t (half, r, a), b_t (half, r, b) half-population factors with
    innermost stride 1 (padded outer strides allowed), scores (n,) raw scores ->
    (g_raw, g_ones), each (a, b): g_raw = sum_i (s_i + s_{half+i}) A_i (x) B_i,
    g_ones = 2 * sum_i A_i (x) B_i.  The reference's `2a <= 256` limit does not apply."""
    return ops.einsum_pair(a_t, b_t, scores)


def prng_normal_half(out: torch.Tensor, mean: float, std: float, seeds: Sequence[int]) -> None:
    """oxide.rs:233-275: fill the contiguous 1-D tensor `out` (length a multiple of
    N_VALUES_PER_THREAD) with N(mean, std) from the hybrid Tausworthe stream, with the four
    seed words passed in instead of being drawn from the wall clock (oxide.rs:205-223)."""
    if out.dim() != 1 or not out.is_contiguous():
        raise ValueError("prng_normal_half: out must be a contiguous 1-D tensor (oxide.rs:225-232)")
    if out.numel() % N_VALUES_PER_THREAD:
        raise ValueError("prng_normal_half: length must be a multiple of N_VALUES_PER_THREAD")
    ops.prng_normal_half(out.numel() // N_VALUES_PER_THREAD, mean, std, seeds, device=out.device, out=out)
