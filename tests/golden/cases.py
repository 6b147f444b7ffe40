"""Seeded input generators shared by the golden-fixture script and the tests.

Everything is drawn from a CPU ``torch.Generator`` so the same tensors appear on any
machine; each fixture also stores a checksum of its inputs to detect drift.
"""
from __future__ import annotations

import torch


def gca_gathered_case(seed: int, z: int, hq: int, hkv: int, k: int, s: int = 64, l: int = 64,
                      d: int = 64, std: float = 0.5, dtype=torch.float32):
    """Inputs shaped like the reference's own op test (``ltriton/gca.py:902-908``):
    q (Z,Hq,S,d), k/v (Z,Hkv,K,L,d) ~ N(0, std), weights = softmax(U[0,1)), dout ~ N(0,1)."""
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(z, hq, s, d, generator=g) * std).to(dtype)
    kk = (torch.randn(z, hkv, k, l, d, generator=g) * std).to(dtype)
    v = (torch.randn(z, hkv, k, l, d, generator=g) * std).to(dtype)
    w = torch.softmax(torch.rand(z, k, generator=g).to(dtype).float(), dim=-1).to(dtype)
    dout = torch.randn(z, hq, s, d, generator=g).to(dtype)
    return q, kk, v, w, dout


def causal_indices(g: torch.Generator, n: int, c: int, k: int):
    """Query chunk j in [1, C) draws min(K, j-1) distinct ids uniformly from [0, j-1);
    the remaining slots are padding (index -1, score -inf).  Returns (N, C-1, K) int64
    indices and float32 scores."""
    idx = torch.full((n, c - 1, k), -1, dtype=torch.int64)
    scores = torch.randn(n, c - 1, k, generator=g)
    for b in range(n):
        for j in range(1, c):
            m = min(k, j - 1)
            if m > 0:
                idx[b, j - 1, :m] = torch.randperm(j - 1, generator=g)[:m]
    scores = torch.where(idx < 0, torch.full_like(scores, float('-inf')), scores)
    return idx, scores


def gca_indexed_case(seed: int, n: int, c: int, h: int, k: int, s: int = 64, d: int = 64,
                     dtype=torch.float32, zero_landmark: bool = True):
    """The benchmark's input recipe: q, caches, upstream grad ~ N(0,1); uniform causal
    retrieved ids; weights = softmax over the valid slots of N(0,1) scores (all-padding
    rows get zero weights).  Caches are token-major (N, C, L, H*d) like the model's."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(n, c - 1, h, s, d, generator=g).to(dtype)
    kc = torch.randn(n, c, s, h * d, generator=g).to(dtype)
    vc = torch.randn(n, c, s, h * d, generator=g).to(dtype)
    if zero_landmark:
        kc[:, :, -1, :] = 0
        vc[:, :, -1, :] = 0
    idx, scores = causal_indices(g, n, c, k)
    w = torch.nan_to_num(torch.softmax(scores, dim=-1), nan=0.0)
    dout = torch.randn(n, c - 1, h, s, d, generator=g).to(dtype)
    return q, kc, vc, idx, w, dout


def landmark_case(seed: int, n: int, cq: int, e: int, d: int = 768, std: float = 1.0):
    """Query landmarks (N, Cq, D) and cached landmarks (N, E, D), bf16-representable."""
    g = torch.Generator().manual_seed(seed)
    lq = (torch.randn(n, cq, d, generator=g) * std).bfloat16()
    lk = (torch.randn(n, e, d, generator=g) * std).bfloat16()
    return lq, lk


def checksum(*tensors) -> float:
    return float(sum(t.double().sum().item() for t in tensors))
