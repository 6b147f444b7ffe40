"""Landmark retrieval: host-side mirror of the reference's retrieval layer.

* ``lmk_score_topk``            -- one fused CUDA pass for ``einsum -> masked_fill -> (+noise)
  -> topk -> softmax -> nan_to_num`` (``model/DRT.py:612-627`` and the decode-time block
  ``:836-845``).
* ``perform_batch_retrieval``   -- same return value as ``DRT._perform_batch_retrieval``
  (``model/DRT.py:609-641``): gathered ``(chunk_k, chunk_v, chunk_weights, indices)``.  It
  exists for drop-in compatibility; the fast path is ``retrieve`` + ``gca.gca_indexed``,
  which never gathers.
* ``decode_retrieval``          -- the chunk-boundary step of generation (``:836-849``).

Selection is canonical: float32 scores summed in one fixed order, ties to the lower chunk
id, padding slots reported as index -1 / weight 0 (``torch.topk`` leaves arbitrary masked
ids there).  ``score_round='bf16'`` reproduces the rounding the reference sees under
autocast (bf16 einsum output, bf16 division) for the selection.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import NamedTuple, Optional

import torch

from . import _lib


class Retrieval(NamedTuple):
    keys: torch.Tensor       # (R.., K) int64 view of the packed uint64 candidates, descending
    indices: torch.Tensor    # (R.., K) int32 global chunk ids, -1 = padding
    scores: torch.Tensor     # (R.., K) float32 noise-free scores
    weights: torch.Tensor    # (R.., K) float32 softmax over valid slots, padding 0
    n_valid: torch.Tensor    # (R..)    int32


def _bf16_rows(t: torch.Tensor, require_bf16: bool = False) -> torch.Tensor:
    """The scan kernel reads bf16 landmarks.  Landmarks in another dtype are ROUNDED to bf16 first:
    that is what the reference's scoring einsum sees under the trainer's bf16 autocast
    (``trainer/slidewindow_trainer.py:198``, ``model/DRT.py:612``), but a float32 run of the
    reference scores in float32 and may pick another chunk on a near tie.  ``require_bf16``
    turns the rounding into an error."""
    if t.dtype != torch.bfloat16:
        if require_bf16:
            raise ValueError(f"landmarks are {t.dtype}: the scan kernel scores bf16 landmarks and would round them "
                             "(pass bf16 tensors, or drop require_bf16 to accept the rounding)")
        t = t.to(torch.bfloat16)
    return t if t.stride(-1) == 1 else t.contiguous()


def lmk_score_topk(lmk_q: torch.Tensor, lmk_k: torch.Tensor, topk: int, *, q_pos0: Optional[int] = None,
                   e_base: int = 0, noise: Optional[torch.Tensor] = None, head_dim: int = 0,
                   score_round: str = "fp32", splits: int = 0, require_bf16: bool = False) -> Retrieval:
    """lmk_q (N, Cq, D), lmk_k (N, E, D) -> top-``topk`` cached chunks per query row.

    Row ``i`` sees cached chunk ``e`` iff ``e_base + e < q_pos0 + i``; the default
    ``q_pos0 = E - Cq`` is the reference's causal chunk mask (``model/DRT.py:590-607``).
    ``head_dim`` = 64 switches to one score / one top-k per head (outputs (N, Cq, H, K)).
    Landmarks that are not bf16 are rounded to bf16 before scoring (see ``_bf16_rows``);
    ``require_bf16=True`` raises instead.
    """
    if not (lmk_q.is_cuda and lmk_k.is_cuda):
        raise RuntimeError("landmark retrieval runs on CUDA tensors only (there is no CPU path)")
    if lmk_q.dim() != 3 or lmk_k.dim() != 3 or lmk_q.shape[0] != lmk_k.shape[0] or lmk_q.shape[2] != lmk_k.shape[2]:
        raise ValueError("expected lmk_q (N, Cq, D) and lmk_k (N, E, D)")
    lq, lk = _bf16_rows(lmk_q.detach(), require_bf16), _bf16_rows(lmk_k.detach(), require_bf16)
    n, cq, d = lq.shape
    e = lk.shape[1]
    heads = d // head_dim if head_dim else 1
    rows_shape = (n, cq, heads) if head_dim else (n, cq)
    dev = lq.device
    keys = torch.empty(rows_shape + (topk,), dtype=torch.int64, device=dev)
    indices = torch.empty(rows_shape + (topk,), dtype=torch.int32, device=dev)
    scores = torch.empty(rows_shape + (topk,), dtype=torch.float32, device=dev)
    weights = torch.empty(rows_shape + (topk,), dtype=torch.float32, device=dev)
    n_valid = torch.empty(rows_shape, dtype=torch.int32, device=dev)
    if n * cq == 0:
        return Retrieval(keys, indices, scores, weights, n_valid)
    a = _lib.LmkTopkArgs()
    a.lmk_q, a.lmk_k = lq.data_ptr(), lk.data_ptr()
    if noise is not None:
        noise = noise.to(torch.float32).contiguous()
        if noise.shape != (n, cq, e):
            raise ValueError("noise must be (N, Cq, E)")
        a.noise = noise.data_ptr()
    a.out_keys, a.out_indices, a.out_scores = keys.data_ptr(), indices.data_ptr(), scores.data_ptr()
    a.out_weights, a.out_nvalid = weights.data_ptr(), n_valid.data_ptr()
    a.q_batch_stride, a.q_row_stride = lq.stride(0), lq.stride(1)
    a.k_batch_stride, a.k_row_stride = lk.stride(0), lk.stride(1)
    a.q_pos0 = (e - cq) if q_pos0 is None else int(q_pos0)
    a.e_base = int(e_base)
    a.N, a.Cq, a.E, a.D, a.K = n, cq, e, d, int(topk)
    a.head_dim = int(head_dim)
    a.score_round = {"fp32": 0, "bf16": 1}[score_round]
    a.splits = int(splits)
    with torch.cuda.device(dev):
        nbytes = _lib.lib().lmk_topk_workspace_bytes(C.byref(a))
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
        a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
        _lib.call("lmk_score_topk", C.byref(a), torch.cuda.current_stream().cuda_stream)
    return Retrieval(keys, indices, scores, weights, n_valid)


def merge_topk(keys: torch.Tensor, topk: int) -> Retrieval:
    """keys (..., P) packed candidates (int64 view of uint64, 0 = empty, any order) ->
    the ``topk`` best per row, identical on every caller given identical input."""
    if not keys.is_cuda:
        raise RuntimeError("merge_topk runs on CUDA tensors only")
    keys = keys.contiguous()
    rows_shape = tuple(keys.shape[:-1])
    r = int(math.prod(rows_shape)) if rows_shape else 1
    dev = keys.device
    out_keys = torch.empty(rows_shape + (topk,), dtype=torch.int64, device=dev)
    indices = torch.empty(rows_shape + (topk,), dtype=torch.int32, device=dev)
    scores = torch.empty(rows_shape + (topk,), dtype=torch.float32, device=dev)
    weights = torch.empty(rows_shape + (topk,), dtype=torch.float32, device=dev)
    n_valid = torch.empty(rows_shape, dtype=torch.int32, device=dev)
    a = _lib.LmkMergeArgs()
    a.keys, a.out_keys, a.out_indices = keys.data_ptr(), out_keys.data_ptr(), indices.data_ptr()
    a.out_scores, a.out_weights, a.out_nvalid = scores.data_ptr(), weights.data_ptr(), n_valid.data_ptr()
    a.R, a.P, a.K = r, keys.shape[-1], int(topk)
    with torch.cuda.device(dev):
        _lib.call("lmk_topk_merge", C.byref(a), torch.cuda.current_stream().cuda_stream)
    return Retrieval(out_keys, indices, scores, weights, n_valid)


def differentiable_weights(lmk_q: torch.Tensor, lmk_k: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """Retrieval weights as a differentiable function of the landmarks (the reference gets
    this from autograd through ``softmax(scores.gather(...))``, ``model/DRT.py:626``): the
    K selected landmarks per row are gathered and re-scored in torch; padding slots get 0."""
    n, cq, d = lmk_q.shape
    idx = indices.clamp(min=0).long()
    batch = torch.arange(n, device=indices.device).view(n, 1, 1)
    sel = lmk_k[batch, idx]                                       # (N, Cq, K, D)
    s = torch.einsum('ncd,nckd->nck', lmk_q, sel.to(lmk_q.dtype)) / math.sqrt(d)
    s = s.float().masked_fill(indices < 0, float('-inf'))
    return torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0)


def retrieve(lmk_q: torch.Tensor, chunk_kvs, topk: int, *, training: bool = False,
             noise: Optional[torch.Tensor] = None, score_round: str = "fp32"):
    """Fast path of ``DRT._perform_batch_retrieval``: returns ``(indices, weights)`` of shape
    (N, Cq-1, K) for query chunks 1..Cq-1 (row i serves query chunk i+1, the last row is
    dropped, ``model/DRT.py:629``) plus the full-row result, without gathering K/V."""
    past = chunk_kvs.past_lmk_embeds
    if training and noise is None:
        # Gumbel noise as in model/DRT.py:616-620
        noise = -torch.empty(lmk_q.shape[0], lmk_q.shape[1], past.shape[1], device=lmk_q.device).exponential_().log()
    res = lmk_score_topk(lmk_q, past, topk, noise=noise, score_round=score_round)
    if lmk_q.requires_grad or past.requires_grad:
        weights = differentiable_weights(lmk_q, past, res.indices)
    else:
        weights = res.weights
    return res.indices[:, :-1], weights[:, :-1], res._replace(weights=weights)


def perform_batch_retrieval(lmk_embs: torch.Tensor, chunk_kvs, group_idx: int, *, num_heads: int,
                            chunk_topk: int, training: bool = False, use_cache: bool = False,
                            noise: Optional[torch.Tensor] = None, score_round: str = "fp32"):
    """Same contract as ``DRT._perform_batch_retrieval`` (``model/DRT.py:609-641``).

    Returns ``(chunk_k, chunk_v, chunk_weights, indices)`` with chunk_k/v
    ``(N*(Cq-1), h, K, S, d)``, chunk_weights ``(N*(Cq-1), K)`` and indices ``(N, Cq, K)``
    int64, K = min(E, chunk_topk).  Padding slots carry index 0 and weight 0 (the reference
    leaves an arbitrary masked id there, also with weight 0).
    """
    from .modules import preprocess_chunk_kv_cache
    past = chunk_kvs.past_lmk_embeds
    e = past.shape[1]
    k = min(e, chunk_topk)
    _, _, res = retrieve(lmk_embs, chunk_kvs, k, training=training, noise=noise, score_round=score_round)
    indices = res.indices.clamp(min=0).long()
    weights = res.weights
    idx_flat = indices[:, :-1].reshape(indices.shape[0], -1)
    rk, rv = chunk_kvs.retrieve_chunks(idx_flat)
    chunk_k, chunk_v, chunk_w = preprocess_chunk_kv_cache(rk, rv, weights[:, :-1], num_heads)
    if use_cache and not training:
        chunk_kvs.update_current_retrieved_chunk(res.indices, weights, group_idx)
    return chunk_k, chunk_v, chunk_w, indices


def decode_retrieval(hidden_last: torch.Tensor, chunk_kvs, group_idx: int, chunk_topk: int,
                     score_round: str = "fp32"):
    """Chunk-boundary retrieval while generating (``model/DRT.py:836-849``): the landmark
    position's hidden state (N, 1, D) is scored against every cached landmark except the
    chunk that was just appended; the winners become the current retrieved chunks."""
    past = chunk_kvs.past_lmk_embeds
    k = min(past.shape[1], chunk_topk)
    res = lmk_score_topk(hidden_last, past, k, score_round=score_round)
    chunk_kvs.update_current_retrieved_chunk(res.indices[:, -1], res.weights[:, -1:], group_idx)
    return res
