"""Seeded degenerate-logit inputs for the top-k selectors, rebuilt from the recipe of the reference's
RouterTopKParityTests (Tests/Mference/Core/Kernels/MoE/RouterTopKParityTests.swift:22-23, 36-47, 61-75, 109-127):
one SplitMix64 stream per expert count, four logit patterns cycling over twelve trials."""
import math

import numpy as np

from oracle import oracle as O

EXPERT_COUNTS = [8, 16, 24, 33, 100, 128, 168, 255, 256]
TRIALS = 12
ROUTE_SCALE = 2.5
F = np.float32


class Rng:
    """Sequential view of a SplitMix64 stream."""

    def __init__(self, seed):
        self.seed, self.i = seed & 0xFFFFFFFFFFFFFFFF, 0

    def next(self):
        v = O.splitmix_at(self.seed, self.i)
        self.i += 1
        return v

    def uniform(self, lo, hi):
        u = F(self.next() >> 40) / F(1 << 24)
        return F(lo) + (F(hi) - F(lo)) * u


def _round_away(x):
    return F(math.floor(abs(float(x)) + 0.5) * (1 if x >= 0 else -1))


def logits_for(count, trial, rng):
    kind = trial % 4
    if kind == 0:
        return [rng.uniform(-4.0, 4.0) for _ in range(count)]
    if kind == 1:   # coarse quantisation: many exact duplicates
        return [_round_away(rng.uniform(-3.0, 3.0) * F(4)) / F(4) for _ in range(count)]
    if kind == 2:   # three levels: the top-k boundary always lands on a tie run
        levels = [F(1.5), F(0.5), F(-0.5)]
        return [levels[rng.next() % 3] for _ in range(count)]
    return [F(0.75)] * count   # all equal: pure index order


def k8_inputs(num_experts):
    """Yields (trial, logits f32[E], per-expert scale f32[E]) for the softmax top-8 selector."""
    rng = Rng(0x5EED0001 + num_experts)
    for trial in range(TRIALS):
        lg = logits_for(num_experts, trial, rng)
        scale = [rng.uniform(0.6, 1.4) for _ in range(num_experts)]
        yield trial, np.array(lg, dtype=F), np.array(scale, dtype=F)


def k6_inputs(num_experts):
    """Yields (trial, logits f32[E], correction bias f32[E]) for the sqrt-softplus top-6 selector."""
    rng = Rng(0x5EED0002 + num_experts)
    for trial in range(TRIALS):
        lg = logits_for(num_experts, trial, rng)
        if trial % 3 == 0:   # duplicated biases: a second source of exact ties
            bias = [F((i // 7) % 4) * F(0.25) for i in range(num_experts)]
        else:
            bias = [rng.uniform(-0.3, 0.3) for _ in range(num_experts)]
        yield trial, np.array(lg, dtype=F), np.array(bias, dtype=F)
