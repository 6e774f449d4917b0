"""Regenerates tests/golden/router_topk_cases.json.

The reference pins its top-k selectors with seeded degenerate logits (continuous, coarsely quantised, three
levels, all equal) over nine expert counts (Tests/Mference/Core/Kernels/MoE/RouterTopKParityTests.swift:22-23,
109-127).  This script rebuilds those inputs from the same seeds and patterns and records the answer given by an
independent definition of the selection — a stable sort by (score descending, expert index ascending) — so
that the oracle and the CUDA selector are both checked against something that is neither of them.

Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

sys.path.insert(0, os.path.join(ROOT, "tests"))
from router_fixtures import EXPERT_COUNTS, ROUTE_SCALE, TRIALS, k6_inputs, k8_inputs  # noqa: E402

F = np.float32


def stable_topk(scores, k):
    order = sorted(range(len(scores)), key=lambda e: (-float(scores[e]), e))[:k]
    return order + [0] * (k - len(order)), len(order)


def sqrtsoftplus(x):
    x = F(x)
    sp = max(x, F(0)) + np.log(F(1) + np.exp(-abs(x)), dtype=F)
    return F(np.sqrt(F(sp)))


def main():
    cases = []
    for ne in EXPERT_COUNTS:
        for trial, lg, scale in k8_inputs(ne):
            idx, filled = stable_topk(lg, 8)
            top = [lg[e] if i < filled else F(-np.inf) for i, e in enumerate(idx)]
            ex = [F(np.exp(F(s - top[0]))) for s in top]
            tot = F(0)
            for v in ex:
                tot = F(tot + v)
            sc_bf16 = O.bf16_to_f32(O.f32_to_bf16(scale))
            w = [float(F(F(ex[i] / tot) * sc_bf16[idx[i]])) for i in range(8)]
            cases.append(dict(mode="softmax_k8", num_experts=ne, trial=trial, indices=idx, weights=w))
        for trial, lg, bias in k6_inputs(ne):
            sel = [F(sqrtsoftplus(lg[e]) + bias[e]) for e in range(ne)]
            idx, _ = stable_topk(sel, 6)
            sc = [sqrtsoftplus(lg[e]) for e in idx]
            tot = F(0)
            for v in sc:
                tot = F(tot + v)
            inv = F(F(ROUTE_SCALE) / F(tot + F(1e-20)))
            w = [float(F(s * inv)) for s in sc]
            cases.append(dict(mode="sqrtsoftplus_k6", num_experts=ne, trial=trial, indices=idx, weights=w))
    out = dict(_comment="expected selections for the seeded degenerate-logit fixtures; see make_golden.py",
               expert_counts=EXPERT_COUNTS, trials=TRIALS, route_scale=ROUTE_SCALE, cases=cases)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "router_topk_cases.json")
    with open(path, "w") as fh:
        json.dump(out, fh)
    print(path, len(cases))


if __name__ == "__main__":
    main()
