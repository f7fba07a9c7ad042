"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

The reference measures this path on uniform-random codes at model shapes
(benchmarks/bench_e8p_m1.py:50-63 of the reference); these generators keep that method.  Every
generator rejects a seed that leaves a tie at the top-k cut, so expert selection is well defined.
"""

from __future__ import annotations

import numpy as np
import torch


def projection(rng, experts, out, inp, group=None, code_bits=16):
    """Uniform codes and per-group fp16 scales 0.02 * U(0.5, 1.5)."""
    group = inp if group is None else group
    hi = 1 << code_bits
    codes = rng.integers(0, hi, (experts, out, inp // 8), dtype=np.uint16 if code_bits == 16 else np.uint8)
    scales = (0.02 * rng.uniform(0.5, 1.5, (experts, out, inp // group))).astype(np.float16)
    return codes, scales


def layer(seed=0, experts=384, hidden=4096, inter=2048, group_hidden=None, group_inter=None):
    """One MoE layer: gate/up [inter x hidden], down [hidden x inter], router bf16 N(0, 0.02^2)."""
    rng = np.random.default_rng(seed)
    w1 = projection(rng, experts, inter, hidden, group_hidden)
    w3 = projection(rng, experts, inter, hidden, group_hidden)
    w2 = projection(rng, experts, hidden, inter, group_inter)
    router = torch.from_numpy(rng.normal(scale=0.02, size=(experts, hidden)).astype(np.float32)).to(torch.bfloat16)
    return dict(w1=w1, w3=w3, w2=w2, router=router, experts=experts, hidden=hidden, inter=inter)


def tokens(seed, count, hidden):
    rng = np.random.default_rng(seed)
    return torch.from_numpy(rng.normal(size=(count, hidden)).astype(np.float32)).to(torch.bfloat16)


def residual_tier(seed, rows, hidden, inter):
    """8-bit residual codes with a flat fp16 scale of 0.005 per row."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, (o, i) in (("w1", (inter, hidden)), ("w3", (inter, hidden)), ("w2", (hidden, inter))):
        codes = rng.integers(0, 256, (rows, o, i // 8), dtype=np.uint8)
        out[name] = (codes, np.full((rows, o, 1), 0.005, dtype=np.float16))
    return out
