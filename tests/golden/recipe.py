"""Seeded input recipe shared by the fixture generator and the tests.

The fixtures store a digest of these inputs instead of the inputs themselves;
a test that regenerates different bits (a changed random generator) fails on
the digest before it compares anything else.
"""
from __future__ import annotations

import hashlib

import numpy as np
import torch


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        if isinstance(a, torch.Tensor):
            a = a.contiguous()
            a = a.view(torch.int16).numpy() if a.dtype in (torch.bfloat16, torch.float16) else a.numpy()
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def make_inputs(*, seed, hq, hkv, tokens, appends, n_queries, dtype=torch.bfloat16, outliers=True):
    """K/V ~ N(0,1); key channels scaled by per-(head, channel) lognormal(0,1)
    factors when ``outliers``; appended tokens and queries from the same stream."""
    g = torch.Generator().manual_seed(int(seed))
    key = torch.randn(hkv, tokens, 128, generator=g)
    if outliers:
        key = key * torch.exp(torch.randn(hkv, 1, 128, generator=g))
    key = key.to(dtype)
    value = torch.randn(hkv, tokens, 128, generator=g).to(dtype)
    new_k = torch.randn(appends, hkv, 128, generator=g)
    if outliers:
        new_k = new_k * torch.exp(torch.randn(1, hkv, 128, generator=g))
    new_k = new_k.to(dtype)
    new_v = torch.randn(appends, hkv, 128, generator=g).to(dtype)
    queries = torch.randn(n_queries, 1, hq, 128, generator=g).to(dtype)
    return key, value, new_k, new_v, queries
