"""CPU oracle for landmark scoring, causal chunk mask, top-k and retrieval weights.
TEST INFRASTRUCTURE ONLY -- never imported by the product path.

What it follows in the reference (paths relative to the reference project):

* scores      -- ``model/DRT.py:612`` / ``:838``: dot product of a query landmark with every
  cached landmark, divided by sqrt(hidden size).
* mask        -- ``model/DRT.py:590-607``: query row ``i`` of ``Cq`` rows over ``E`` cached
  chunks has chunk id ``E - Cq + i`` and sees only chunks with a smaller id.
* top-k       -- ``model/DRT.py:623-625`` (``k = min(E, topk)``, noise added for selection
  only) and decode ``:842-843``.
* weights     -- ``model/DRT.py:626-627``: softmax over the noise-free selected scores,
  NaN (all-masked row) -> 0.

``torch.topk`` does not define which of two equal scores wins and returns arbitrary ids for
masked (-inf) slots, so "bit-exact indices" needs a canonical statement.  This oracle defines
it: scores are float32 sums in ONE fixed order (below), ordered by (score descending, index
ascending); masked entries are never selected; slots beyond the number of visible chunks are
padding (index -1, weight 0).  ``torch_reference_retrieval`` is the literal torch sequence,
used to check set-equality on tie-free rows.

Fixed reduction order (``canonical_scores``): the D-vector is cut in 8-element pieces;
piece ``c`` belongs to lane ``c % 32`` of 32 lanes and is visited in increasing ``c``; a lane
adds its products one by one (float32, products of bf16 values are exact); the 32 lane sums
are combined by a butterfly: for off in 16, 8, 4, 2, 1: s[l] += s[l ^ off].  In per-head mode
the butterfly stops inside the ``head_dim/8`` lanes that hold one head.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np

LANES = 32
PIECE = 8


def _bf16_round(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 -> float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    out = ((u + r) & np.uint32(0xFFFF0000)).astype(np.uint32)
    nan = np.isnan(x)
    res = out.view(np.float32).copy()
    res[nan] = np.nan
    return res


def canonical_scores(lq: np.ndarray, lk: np.ndarray, *, head_dim: int = 0,
                     score_round: str = "fp32") -> np.ndarray:
    """lq (Cq, D), lk (E, D): bf16-representable float32.  Returns (Cq, E) float32 in
    per-sequence mode (head_dim == 0) or (Cq, H, E) in per-head mode."""
    lq = np.ascontiguousarray(lq, dtype=np.float32)
    lk = np.ascontiguousarray(lk, dtype=np.float32)
    cq, d = lq.shape
    e = lk.shape[0]
    assert d % PIECE == 0
    pieces = d // PIECE
    passes = (pieces + LANES - 1) // LANES
    acc = np.zeros((cq, e, LANES), dtype=np.float32)
    for p in range(passes):
        lo = p * LANES
        n_l = min(LANES, pieces - lo)
        for j in range(PIECE):
            cols = (lo + np.arange(n_l)) * PIECE + j
            prod = lq[:, None, cols] * lk[None, :, cols]          # exact in float32 for bf16 inputs
            acc[:, :, :n_l] = acc[:, :, :n_l] + prod
    lane = np.arange(LANES)
    if head_dim == 0:
        offs = (16, 8, 4, 2, 1)
        scale = np.float32(1.0 / math.sqrt(d))
    else:
        lph = head_dim // PIECE
        assert lph in (1, 2, 4, 8, 16, 32) and d % head_dim == 0
        offs = tuple(o for o in (16, 8, 4, 2, 1) if o < lph)
        scale = np.float32(1.0 / math.sqrt(head_dim))
    if head_dim == 0:
        for off in offs:
            acc = acc + acc[:, :, lane ^ off]
        raw = acc[:, :, 0]
    else:
        # every pass holds LANES/lph heads; redo per pass because lanes are reused across passes
        lph = head_dim // PIECE
        heads = d // head_dim
        raw = np.zeros((cq, heads, e), dtype=np.float32)
        for p in range(passes):
            a = np.zeros((cq, e, LANES), dtype=np.float32)
            lo = p * LANES
            n_l = min(LANES, pieces - lo)
            for j in range(PIECE):
                cols = (lo + np.arange(n_l)) * PIECE + j
                a[:, :, :n_l] = a[:, :, :n_l] + lq[:, None, cols] * lk[None, :, cols]
            for off in offs:
                a = a + a[:, :, lane ^ off]
            for g in range(n_l // lph):
                raw[:, (lo // lph) + g, :] = a[:, :, g * lph]
    if score_round == "bf16":
        # the reference under autocast: the einsum result is rounded to bf16, and so is the
        # scaled score (model/DRT.py:612 inside trainer/slidewindow_trainer.py:198)
        return _bf16_round(_bf16_round(raw) * scale)
    return (raw * scale).astype(np.float32)


def visible_limit(cq: int, e_total: int) -> np.ndarray:
    """Row i of Cq query landmarks sees cached chunks with id < E - Cq + i (DRT.py:596-600)."""
    return (e_total - cq) + np.arange(cq)


def _orderable(score: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(score, dtype=np.float32).view(np.uint32).astype(np.uint64)
    neg = (u >> np.uint64(31)) == 1
    return np.where(neg, (~u) & np.uint64(0xFFFFFFFF), u | np.uint64(0x80000000))


def pack_keys(score: np.ndarray, index: np.ndarray) -> np.ndarray:
    """uint64 key whose integer order is (score descending wins, lower index wins)."""
    return (_orderable(score) << np.uint64(32)) | (np.uint64(0xFFFFFFFF) - index.astype(np.uint64))


def unpack_keys(keys: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    keys = keys.astype(np.uint64)
    idx = (np.uint64(0xFFFFFFFF) - (keys & np.uint64(0xFFFFFFFF))).astype(np.int64)
    o = (keys >> np.uint64(32)).astype(np.uint32)
    neg = (o >> np.uint32(31)) == 0
    u = np.where(neg, ~o, o & np.uint32(0x7FFFFFFF)).astype(np.uint32)
    score = u.view(np.float32)
    empty = keys == 0
    idx = np.where(empty, -1, idx)
    score = np.where(empty, -np.inf, score).astype(np.float32)
    return score, idx


def canonical_topk(scores: np.ndarray, limit: np.ndarray, topk: int,
                   noise: Optional[np.ndarray] = None, e_base: int = 0
                   ) -> Tuple[np.ndarray, np.ndarray, np.ndarray, np.ndarray]:
    """scores (R, E) float32; limit (R,) = number of visible global chunk ids per row.

    Returns (indices (R, K) int64 global ids, -1 = padding; selected noise-free scores
    (R, K) float32; weights (R, K) float32; n_valid (R,))."""
    r, e = scores.shape
    sel = scores if noise is None else (scores + noise.astype(np.float32)).astype(np.float32)
    gidx = e_base + np.arange(e, dtype=np.int64)
    keys = pack_keys(sel, np.broadcast_to(gidx, (r, e)))
    vis = gidx[None, :] < limit[:, None]
    keys = np.where(vis, keys, np.uint64(0))
    k = topk
    order = np.argsort(keys, axis=1, kind="stable")[:, ::-1][:, :k]
    top = np.take_along_axis(keys, order, axis=1)
    if top.shape[1] < k:
        top = np.concatenate([top, np.zeros((r, k - top.shape[1]), dtype=np.uint64)], axis=1)
        order = np.concatenate([order, np.zeros((r, k - order.shape[1]), dtype=order.dtype)], axis=1)
    _, idx = unpack_keys(top)
    valid = top != 0
    clean = np.where(valid, np.take_along_axis(scores, np.clip(order, 0, e - 1), axis=1), -np.inf).astype(np.float32)
    weights = softmax_valid(clean, valid)
    return idx, clean, weights, valid.sum(axis=1).astype(np.int32)


def softmax_valid(clean: np.ndarray, valid: np.ndarray) -> np.ndarray:
    """softmax over the valid slots (DRT.py:626); rows without any valid slot give zeros (:627)."""
    m = np.max(np.where(valid, clean, -np.inf), axis=1, keepdims=True)
    m = np.where(np.isfinite(m), m, 0.0).astype(np.float32)
    ex = np.where(valid, np.exp((clean - m).astype(np.float32)), 0.0).astype(np.float32)
    den = ex.sum(axis=1, keepdims=True, dtype=np.float32)
    return np.where(den > 0, ex / np.where(den > 0, den, 1.0), 0.0).astype(np.float32)


def merge_candidates(keys: np.ndarray, topk: int) -> np.ndarray:
    """keys (R, P) packed uint64 candidates from P/k shards -> (R, k) best keys, descending.
    Identical keys cannot occur for distinct global indices, so the result is unique."""
    s = np.sort(keys.astype(np.uint64), axis=1)[:, ::-1]
    return s[:, :topk]


def torch_reference_retrieval(lq, lk, topk: int, noise=None):
    """Literal torch restatement of ``model/DRT.py:612-627`` for one sequence batch.

    lq (N, Cq, D), lk (N, E, D) torch tensors.  Returns (indices (N, Cq, k), weights)."""
    import torch
    import torch.nn.functional as F
    d = lq.shape[-1]
    scores = torch.einsum('ncd,ned->nce', lq, lk) / math.sqrt(d)
    cq, e = scores.shape[1], scores.shape[2]
    dec = torch.arange(e)[-cq:]
    enc = torch.arange(e)
    visible = dec.unsqueeze(1) > enc.unsqueeze(0)
    scores = scores.masked_fill(~visible, float('-inf'))
    nz = torch.zeros_like(scores) if noise is None else noise
    k = min(e, topk)
    _, indices = torch.topk(scores + nz, dim=2, k=k)
    w = F.softmax(scores.gather(dim=2, index=indices), dim=-1)
    w = torch.nan_to_num(w, nan=0.0)
    return indices, w
