"""CPU oracle for Grouped Cross-Attention (GCA).  TEST INFRASTRUCTURE ONLY.

This file restates, in plain PyTorch on the CPU, the arithmetic of the
reference's GCA operator.  Only the test-suite, the smoke check and the CPU
baseline leg of the benchmark may import it; the product path never does.

What it follows in the reference (paths are relative to the reference project):

* ``gca_gathered``        -- the einsum formulation the reference's own unit test
  uses as ground truth, ``ltriton/gca.py:912-921`` (repeat_interleave for GQA,
  QK^T * scale, softmax over the keys of one chunk, PV, merge of the K per-chunk
  outputs with the retrieval weights).  Gradients come from autograd of that
  expression, exactly like ``ltriton/gca.py:922-926``.
* ``gather_chunks``       -- ``ChunkKVManager.retrieve_chunks``
  (``model/DRT.py:193-199``) followed by
  ``TritonGroupCrossAttention.preprocess_chunk_kv_cache`` (``model/DRT.py:321-332``).
* ``gca_indexed``         -- the two above composed: what the model computes for a
  (cache, indices, weights) triple, including the scatter-add of dK/dV back into the
  cache that autograd performs through the advanced-index gather.
* ``softmax_off_by_one``  -- NOT in the shipped Triton kernel (its ``sm_n`` argument is
  erased by the first online-softmax step, ``ltriton/gca.py:48-49,187``); defined here
  as a softmax over ``[logits, 0]`` whose extra column (weight ``sm_n``) is dropped.
  Parity for this variant is unpinned by any reference test.

Pinning: the golden fixtures in ``tests/golden`` are produced by executing the
reference's own source lines (extracted from the reference checkout by
``tests/golden/make_golden.py``); ``tests/test_oracle.py`` checks this file against
them.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def gca_gathered(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, weights: torch.Tensor,
                 sm_scale: float, *, p_dtype: Optional[torch.dtype] = None,
                 off_by_one: float = 0.0) -> torch.Tensor:
    """GCA over pre-gathered chunks.

    q (Z, Hq, S, d); k, v (Z, Hkv, K, L, d); weights (Z, K) -> (Z, Hq, S, d).
    ``p_dtype`` reproduces the cast of the probabilities before the PV product
    (``ltriton/gca.py:917``: ``.to(dtype)``); ``None`` keeps the working precision.
    ``off_by_one`` > 0 adds a virtual zero logit of that weight to every softmax.
    """
    group = q.shape[1] // k.shape[1]
    k_ = torch.repeat_interleave(k, dim=1, repeats=group)
    v_ = torch.repeat_interleave(v, dim=1, repeats=group)
    p = torch.einsum('zhmd,zhknd->zhkmn', q, k_) * sm_scale
    if off_by_one > 0.0:
        # softmax over [p, 0] with the virtual column weighted by off_by_one, then dropped
        m = torch.clamp(p.amax(dim=-1, keepdim=True), min=0.0)
        e = torch.exp(p - m)
        p = e / (e.sum(dim=-1, keepdim=True) + off_by_one * torch.exp(-m))
    else:
        p = torch.softmax(p, dim=-1)
    if p_dtype is not None:
        p = p.to(p_dtype).to(v_.dtype)
    o_k = torch.einsum('zhkmn,zhknd->zhkmd', p, v_)
    return torch.einsum('zhkmd,zk->zhmd', o_k, weights.to(o_k.dtype))


def gca_lse(q: torch.Tensor, k: torch.Tensor, sm_scale: float, off_by_one: float = 0.0) -> torch.Tensor:
    """Base-2 log-sum-exp per (z, head, slot, row): what the forward saves for the
    backward (``ltriton/gca.py:197,204``), returned as (Z, Hq, K, S)."""
    group = q.shape[1] // k.shape[1]
    k_ = torch.repeat_interleave(k, dim=1, repeats=group)
    s = torch.einsum('zhmd,zhknd->zhkmn', q, k_) * (sm_scale * 1.4426950408889634)
    if off_by_one > 0.0:
        zero = torch.full_like(s[..., :1], math.log2(off_by_one))
        s = torch.cat([s, zero], dim=-1)
    return torch.logsumexp(s * math.log(2.0), dim=-1) / math.log(2.0)


def gather_chunks(k_cache: torch.Tensor, v_cache: torch.Tensor, indices: torch.Tensor,
                  num_kv_heads: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Cache (N, C, L, Hkv*d), indices (N, J, K) -> k, v (N*J, Hkv, K, L, d).

    Follows ``model/DRT.py:193-199`` (advanced-index gather) and ``:328-332``
    (split heads, move them in front of the slot axis).  Negative indices denote
    padding slots; they are clamped to 0 for the gather (their weight must be 0).
    """
    n, j, kk = indices.shape
    idx = indices.clamp(min=0).reshape(n, j * kk).long()
    batch = torch.arange(n, device=indices.device).unsqueeze(1)
    gk = k_cache[batch, idx]            # (N, J*K, L, Hkv*d)
    gv = v_cache[batch, idx]
    l, hd = gk.shape[-2], gk.shape[-1]
    d = hd // num_kv_heads

    def split(t):
        t = t.reshape(n, j, kk, l, num_kv_heads, d)
        return t.permute(0, 1, 4, 2, 3, 5).reshape(n * j, num_kv_heads, kk, l, d)

    return split(gk), split(gv)


def gca_indexed(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                indices: torch.Tensor, weights: torch.Tensor, sm_scale: float, *,
                p_dtype: Optional[torch.dtype] = None, off_by_one: float = 0.0) -> torch.Tensor:
    """q (N, J, Hq, S, d); caches (N, C, L, Hkv*d); indices, weights (N, J, K).

    Returns (N, J, Hq, S, d).  Padding slots (index < 0) contribute nothing.
    """
    n, j, hq, s, d = q.shape
    hkv = k_cache.shape[-1] // d
    gk, gv = gather_chunks(k_cache, v_cache, indices, hkv)
    w = torch.where(indices < 0, torch.zeros_like(weights), weights).reshape(n * j, -1)
    o = gca_gathered(q.reshape(n * j, hq, s, d), gk, gv, w, sm_scale,
                     p_dtype=p_dtype, off_by_one=off_by_one)
    return o.reshape(n, j, hq, s, d)


def gca_indexed_grads(q, k_cache, v_cache, indices, weights, sm_scale, dout, *,
                      p_dtype=None, off_by_one: float = 0.0, work_dtype=torch.float32):
    """Forward + autograd backward of ``gca_indexed`` in ``work_dtype``.

    Returns (o, dq, dk_cache, dv_cache, dw).  dK/dV are in cache layout: the sum over all
    (query chunk, slot) pairs that retrieved a chunk, which is what the reference obtains
    through autograd of its gather (``index_put_(accumulate=True)``)."""
    q_ = q.detach().to(work_dtype).requires_grad_()
    k_ = k_cache.detach().to(work_dtype).requires_grad_()
    v_ = v_cache.detach().to(work_dtype).requires_grad_()
    w_ = weights.detach().to(work_dtype).requires_grad_()
    o = gca_indexed(q_, k_, v_, indices, w_, sm_scale, p_dtype=p_dtype, off_by_one=off_by_one)
    o.backward(dout.to(work_dtype))
    dw = w_.grad if w_.grad is not None else torch.zeros_like(w_)
    dw = torch.where(indices < 0, torch.zeros_like(dw), dw)
    return o.detach(), q_.grad, k_.grad, v_.grad, dw


def gca_gathered_grads(q, k, v, weights, sm_scale, dout, *, p_dtype=None, off_by_one: float = 0.0,
                       work_dtype=torch.float32):
    """Forward + autograd backward of ``gca_gathered`` (``ltriton/gca.py:912-926``)."""
    q_ = q.detach().to(work_dtype).requires_grad_()
    k_ = k.detach().to(work_dtype).requires_grad_()
    v_ = v.detach().to(work_dtype).requires_grad_()
    w_ = weights.detach().to(work_dtype).requires_grad_()
    o = gca_gathered(q_, k_, v_, w_, sm_scale, p_dtype=p_dtype, off_by_one=off_by_one)
    o.backward(dout.to(work_dtype))
    return o.detach(), q_.grad, k_.grad, v_.grad, w_.grad


def zero_landmark_rows(chunk_k: torch.Tensor, chunk_v: torch.Tensor):
    """The model's effective softmax-off-by-one: the landmark (last) row of every chunk of
    K and V is zeroed before it enters the cache (``model/DRT.py:771-781``)."""
    chunk_k = chunk_k.clone()
    chunk_v = chunk_v.clone()
    chunk_k[..., -1, :] = 0
    chunk_v[..., -1, :] = 0
    return chunk_k, chunk_v
