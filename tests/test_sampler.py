"""Canonical sampler, summary sampler and repetition penalty (C++ host library)."""
import math

import numpy as np
import torch

from r4dx_b200.runtime.sampler import (Rng, SampleParams, apply_repetition_penalty, row_summary, sample_canonical,
                                        sample_from_summary)


def _reference(logits, p, u):
    l = logits.double().numpy()
    order = sorted(range(len(l)), key=lambda i: (-l[i], i))
    pr = np.exp((l - l.max()) / p.temperature)
    pr = pr / pr.sum()
    ps = pr[order]
    keep = len(order)
    if p.top_k > 0:
        keep = min(keep, p.top_k)
    if p.min_p > 0:
        k = 0
        while k < keep and ps[k] >= p.min_p * ps[0]:
            k += 1
        keep = max(1, k)
    if p.top_p < 1:
        mass = ps[:keep].sum()
        c, k = 0.0, 0
        while k < keep:
            c += ps[k]; k += 1
            if c >= p.top_p * mass:
                break
        keep = k
    kept = ps[:keep].sum()
    c = 0.0
    for i in range(keep):
        c += ps[i]
        if u * kept < c:
            return order[i]
    return order[keep - 1]


def test_canonical_matches_reference_pipeline():
    g = torch.Generator().manual_seed(0)
    for trial in range(40):
        logits = torch.randn(3000, generator=g) * 3
        logits[5] = logits[77]                                  # an exact tie
        p = SampleParams(temperature=[0.7, 1.0, 1.3][trial % 3], top_k=[0, 50, 5][trial % 3],
                         top_p=[1.0, 0.9, 0.5][(trial // 3) % 3], min_p=[0.0, 0.05][(trial // 9) % 2])
        u = float(torch.rand(1, generator=g))
        assert sample_canonical(logits, p, u) == _reference(logits, p, u)


def test_greedy_and_ties():
    l = torch.zeros(100)
    l[40] = l[7] = 2.0
    assert sample_canonical(l, SampleParams(temperature=0.0), 0.3) == 7
    assert sample_canonical(l, SampleParams(temperature=1.0, top_k=1), 0.99) == 7


def test_summary_agrees_or_abstains():
    g = torch.Generator().manual_seed(1)
    proved = 0
    for trial in range(60):
        logits = torch.randn(5000, generator=g) * (4 if trial % 2 else 1)
        p = SampleParams(temperature=0.8, top_k=[0, 40][trial % 2], top_p=[0.95, 1.0][(trial // 2) % 2])
        u = float(torch.rand(1, generator=g))
        tl, ids, lse = row_summary(logits, p.temperature)
        s = sample_from_summary(tl, ids, lse, p, u)
        full = sample_canonical(logits, p, u)
        if s >= 0:
            proved += 1
            assert s == full
    assert proved > 20


def test_rng_is_deterministic_and_uniform():
    a, b = Rng(42), Rng(42)
    xs = [a.next() for _ in range(1000)]
    assert xs == [b.next() for _ in range(1000)]
    assert 0.45 < sum(xs) / 1000 < 0.55 and all(0 <= x < 1 for x in xs)


def test_repetition_penalty():
    l = torch.tensor([2.0, -2.0, 1.0, 0.5])
    apply_repetition_penalty(l, [0, 1, 1, 0], 2.0)
    assert l.tolist() == [1.0, -4.0, 1.0, 0.5]
