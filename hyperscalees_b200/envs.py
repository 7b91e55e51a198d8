"""Host-side mirror of hyperscalees-envs/src/snn_mnist.rs for the pieces on the
population step: Poisson encoding and fitness."""
from __future__ import annotations

from typing import Sequence

import torch

from . import ops

Loglik, Binary = ops.REWARD_LOGLIK, ops.REWARD_BINARY


def poisson_encode(images: torch.Tensor, t: int, seeds: Sequence[int] = (0, 0, 0, 0)) -> torch.Tensor:
    """snn_mnist.rs:144-155: (batch, in_dim) probabilities -> (t, batch, in_dim) 0/1 spikes.

    The reference's CPU version draws from Burn's global RNG and is not
    reproducible (snn_mnist.rs:135-138); this one is the deterministic
    xorshift32 stream of the reference's fused GPU kernel
    (poisson_encode_fused_oxide.rs:61-106) with caller-supplied seed words.
    """
    return ops.poisson_encode(images, t, seeds)


def fitness_from_logits_reward(logits: torch.Tensor, labels: torch.Tensor, reward: int) -> torch.Tensor:
    """snn_mnist.rs:180-201."""
    return ops.fitness(logits, labels.to(torch.int32), reward)


def fitness_from_logits(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """snn_mnist.rs:171-173: the hard 0/1 reward."""
    return fitness_from_logits_reward(logits, labels, Binary)


def accuracy_from_logits(logits: torch.Tensor, labels: torch.Tensor) -> float:
    """snn_mnist.rs:206-212: mean of the 0/1 reward over the batch."""
    hits = fitness_from_logits(logits, labels)
    return float(ops.member_mean(hits, 1, hits.numel()).item())
