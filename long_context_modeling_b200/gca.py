"""Grouped Cross-Attention: host-side mirror of the reference's ``ltriton/gca.py`` boundary.

``attention`` and ``gca_kv_cache`` keep the reference's positional signatures
(``ltriton/gca.py:844`` / ``:846``, called from ``model/DRT.py:380,382``) so a model can
rebind ``model.DRT.gca_attn`` / ``model.DRT.gca_kv_cache`` to them.  ``gca_indexed`` is the
extended entry: it takes the chunk cache and the retrieved indices and never materialises
the gathered copy (``model/DRT.py:193-199`` + ``:321-332`` in the reference); gradients
flow to the cache.

All arithmetic happens in the CUDA library behind the C ABI (``_lib``); this file only
arranges views, strides and autograd bookkeeping.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from ._lib import ALGO_AUTO, ALGO_SIMT, ALGO_TC, ALGO_TC_UNPAIRED  # noqa: F401  (re-exported)

_status_words: Dict[int, torch.Tensor] = {}


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.BF16
    if t.dtype == torch.float32:
        return _lib.F32
    raise ValueError(f"unsupported dtype {t.dtype}: the GCA kernels take bfloat16 or float32")


def _status(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status_words:
        _status_words[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[idx]


def read_status(device=None, clear: bool = True) -> int:
    """Device-side soft status bits accumulated by the kernels (synchronises)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = _status(device)
    val = int(word.item())
    if clear:
        word.zero_()
    return val


_check_after_launch = False


def set_status_checks(enabled: bool) -> None:
    """When enabled, every GCA call of this module reads the device status word after its launch
    (one synchronisation per call) and raises ``GcaError`` if a kernel reported that a bounded
    wait expired (outputs invalid).  Off by default; ``HostGcaPipeline`` always checks, at the
    point where it synchronises anyway."""
    global _check_after_launch
    _check_after_launch = bool(enabled)


def check_status(device=None, clear: bool = True) -> int:
    """Reads the status word (synchronises).  ``STATUS_TIMEOUT`` -- a kernel gave up a bounded
    on-chip wait, its outputs are not valid -- raises ``GcaError``; other bits (a retrieved index
    outside the cache: that slot was skipped) are returned to the caller."""
    bits = read_status(device, clear)
    if bits & _lib.STATUS_TIMEOUT:
        raise _lib.GcaError("a GCA kernel gave up a bounded wait (GCA_STATUS_TIMEOUT): its outputs are not valid")
    return bits


def _maybe_check(device) -> None:
    if _check_after_launch:
        check_status(device)


def _require_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("GCA runs on CUDA tensors only (there is no CPU path)")


def _as_cache5(cache: torch.Tensor, head_dim: int) -> torch.Tensor:
    """(N, C, L, Hkv*D) token-major cache, or already (N, C, L, Hkv, D) -> 5-D view."""
    if cache.dim() == 5:
        return cache
    if cache.dim() != 4 or cache.shape[-1] % head_dim != 0:
        raise ValueError(f"cache must be (N, C, L, Hkv*D) or (N, C, L, Hkv, D), got {tuple(cache.shape)}")
    if cache.stride(-1) != 1:
        cache = cache.contiguous()
    return cache.unflatten(-1, (cache.shape[-1] // head_dim, head_dim))


def _inner_contiguous(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


def _fwd_args(q5, kc5, vc5, idx32, w32, out5, lse, sm_scale, off_by_one, algo) -> _lib.GcaFwdArgs:
    n, j, hq, s, d = q5.shape
    _, c, l, hkv, _ = kc5.shape
    a = _lib.GcaFwdArgs()
    a.q, a.k_cache, a.v_cache = q5.data_ptr(), kc5.data_ptr(), vc5.data_ptr()
    a.indices, a.weights, a.out = idx32.data_ptr(), w32.data_ptr(), out5.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.status = _status(q5.device).data_ptr()
    a.q_stride = _lib.strides4(*q5.stride()[:4])
    a.o_stride = _lib.strides4(*out5.stride()[:4])
    a.k_stride = _lib.strides4(*kc5.stride()[:4])
    a.v_stride = _lib.strides4(*vc5.stride()[:4])
    a.N, a.J, a.Hq, a.Hkv, a.S, a.L, a.D, a.K, a.C = n, j, hq, hkv, s, l, d, idx32.shape[-1], c
    a.dtype = _dtype_code(q5)
    a.algo = algo
    a.sm_scale = float(sm_scale)
    a.off_by_one = float(off_by_one)
    return a


def _check_shapes(q5, kc5, vc5, idx, w):
    if q5.dim() != 5 or kc5.dim() != 5 or vc5.dim() != 5:
        raise ValueError("expected q (N,J,Hq,S,D) and caches (N,C,L,Hkv,D)")
    if kc5.shape != vc5.shape:
        raise ValueError("k_cache and v_cache must have the same shape")
    if q5.dtype != kc5.dtype or q5.dtype != vc5.dtype:
        raise ValueError("q, k_cache and v_cache must share one dtype")
    n, j = q5.shape[0], q5.shape[1]
    if idx.shape[:2] != (n, j) or w.shape != idx.shape or kc5.shape[0] != n:
        raise ValueError(f"indices/weights must be (N, J, K) = ({n}, {j}, K); got {tuple(idx.shape)}, {tuple(w.shape)}")
    if q5.shape[-1] != kc5.shape[-1]:
        raise ValueError("head dims of q and the cache differ")
    if q5.shape[2] % kc5.shape[3] != 0:
        raise ValueError("number of q heads must be a multiple of the number of kv heads")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class _GcaIndexed(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q5, kc5, vc5, idx32, w32, sm_scale, off_by_one, algo, token_major_out=False):
        n, j, hq, s, d = q5.shape
        k = idx32.shape[-1]
        if token_major_out:
            # memory order (n, j, s, h, d): the caller can flatten it to (N, J*S, H*D) for free
            out = torch.empty((n, j, s, hq, d), dtype=q5.dtype, device=q5.device).permute(0, 1, 3, 2, 4)
        else:
            out = torch.empty((n, j, hq, s, d), dtype=q5.dtype, device=q5.device)
        lse = torch.empty((n * j, hq, k, s), dtype=torch.float32, device=q5.device)
        with torch.cuda.device(q5.device):
            a = _fwd_args(q5, kc5, vc5, idx32, w32, out, lse, sm_scale, off_by_one, algo)
            _lib.call("gca_fwd", C.byref(a), _stream())
        _maybe_check(q5.device)
        ctx.save_for_backward(q5, kc5, vc5, idx32, w32, lse)
        ctx.sm_scale, ctx.off_by_one, ctx.algo = sm_scale, off_by_one, algo
        return out

    @staticmethod
    def backward(ctx, dout):
        q5, kc5, vc5, idx32, w32, lse = ctx.saved_tensors
        dq, dk, dv, dw = _backward_call(q5, kc5, vc5, idx32, w32, dout, lse, ctx.sm_scale, ctx.off_by_one, ctx.algo)
        return dq, dk, dv, None, dw, None, None, None, None


BWD_STAGE_INDEX, BWD_STAGE_KV, BWD_STAGE_Q, BWD_STAGE_ALL = 1, 2, 4, 7
BWD_INDEX_BY_SORT = 8          # flag beside BWD_STAGE_INDEX: build the inverse index by radix sort (same bits)


def _backward_call(q5, kc5, vc5, idx32, w32, dout, lse, sm_scale, off_by_one, algo, stages=BWD_STAGE_ALL, bufs=None):
    """One `gca_bwd_stages` call.  `bufs` = (dq, dk, dv, dw, workspace) from an earlier call of the
    same backward (the stages of one backward share their outputs and the inverse index)."""
    dout = _inner_contiguous(dout)
    n, j, hq, s, d = q5.shape
    _, c, l, hkv, _ = kc5.shape
    k = idx32.shape[-1]
    a = _lib.GcaBwdArgs()
    a.q, a.k_cache, a.v_cache = q5.data_ptr(), kc5.data_ptr(), vc5.data_ptr()
    a.indices, a.weights, a.dout, a.lse = idx32.data_ptr(), w32.data_ptr(), dout.data_ptr(), lse.data_ptr()
    a.N, a.J, a.Hq, a.Hkv, a.S, a.L, a.D, a.K, a.C = n, j, hq, hkv, s, l, d, k, c
    a.dtype = _dtype_code(q5)
    a.algo = algo
    a.sm_scale, a.off_by_one = float(sm_scale), float(off_by_one)
    with torch.cuda.device(q5.device):
        if bufs is None:
            dq = torch.empty_like(q5)
            if dq.stride(-1) != 1:
                dq = torch.empty((n, j, hq, s, d), dtype=q5.dtype, device=q5.device)
            dk = torch.empty_like(kc5)
            dv = torch.empty_like(vc5)
            if dk.stride(-1) != 1 or dv.stride(-1) != 1:
                dk = torch.empty(kc5.shape, dtype=kc5.dtype, device=kc5.device)
                dv = torch.empty(vc5.shape, dtype=vc5.dtype, device=vc5.device)
            dw = torch.empty((n, j, k), dtype=torch.float32, device=q5.device)
            nbytes = _lib.lib().gca_bwd_workspace_bytes(C.byref(a))
            ws = torch.empty(nbytes + 256, dtype=torch.uint8, device=q5.device)
        else:
            dq, dk, dv, dw, ws = bufs
        a.dq, a.dk_cache, a.dv_cache, a.dw = dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dw.data_ptr()
        a.status = _status(q5.device).data_ptr()
        a.q_stride = _lib.strides4(*q5.stride()[:4])
        a.do_stride = _lib.strides4(*dout.stride()[:4])
        a.dq_stride = _lib.strides4(*dq.stride()[:4])
        a.k_stride = _lib.strides4(*kc5.stride()[:4])
        a.v_stride = _lib.strides4(*vc5.stride()[:4])
        a.dk_stride = _lib.strides4(*dk.stride()[:4])
        a.dv_stride = _lib.strides4(*dv.stride()[:4])
        a.workspace = (ws.data_ptr() + 255) // 256 * 256
        a.workspace_bytes = ws.numel() - 256
        _lib.call("gca_bwd_stages", C.byref(a), stages, _stream())
    _maybe_check(q5.device)
    if bufs is None and (stages & BWD_STAGE_ALL) != BWD_STAGE_ALL:
        return dq, dk, dv, dw, ws
    return dq, dk, dv, dw


def gca_backward_stages(q, k_cache, v_cache, indices, weights, dout, lse, sm_scale, *, stages=BWD_STAGE_ALL,
                        bufs=None, softmax_off_by_one=False, algo: int = ALGO_AUTO):
    """The backward of `gca_indexed` without autograd, optionally one stage at a time:
    BWD_STAGE_INDEX, then BWD_STAGE_Q, then BWD_STAGE_KV (the dK/dV kernel reads per-row terms
    that the dQ kernel leaves in the workspace).  `stages | BWD_INDEX_BY_SORT` builds the index
    by radix sort.

    q (N, J, Hq, S, D); caches (N, C, L, Hkv*D); dout like q; lse as returned by
    `gca_forward_with_lse`.  A partial call returns (dq, dk, dv, dw, workspace): pass that tuple
    back as `bufs` for the remaining stages.  A full call returns (dq, dk, dv, dw).
    """
    d = q.shape[-1]
    q5, kc5, vc5 = _inner_contiguous(q), _as_cache5(k_cache, d), _as_cache5(v_cache, d)
    _check_shapes(q5, kc5, vc5, indices, weights)
    idx32 = indices.to(torch.int32).contiguous()
    w32 = weights.to(torch.float32).contiguous()
    return _backward_call(q5, kc5, vc5, idx32, w32, dout, lse, sm_scale, 1.0 if softmax_off_by_one else 0.0, algo,
                          stages, bufs)


def gca_indexed(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, indices: torch.Tensor,
                weights: torch.Tensor, sm_scale: float, sm_n: float = 0.0, *,
                softmax_off_by_one: bool = False, algo: int = ALGO_AUTO,
                token_major_out: bool = False) -> torch.Tensor:
    """GCA straight from the chunk cache.

    q (N, J, Hq, S, D); caches (N, C, L, Hkv*D) token-major (the layout of
    ``ChunkKVManager``, ``model/DRT.py:88``) or (N, C, L, Hkv, D); indices (N, J, K) integer,
    negative = padding slot; weights (N, J, K).  Returns (N, J, Hq, S, D) in q's dtype.

    ``sm_n`` is accepted for signature compatibility and, exactly like the reference
    kernels, has no effect unless ``softmax_off_by_one=True``, which adds a virtual zero
    logit of weight ``sm_n`` (default 1 when sm_n == 0) to every per-chunk softmax.
    ``token_major_out`` lays the result out as (n, j, s, h, d) in memory (returned as a
    permuted view of the same logical shape), which is what the output projection wants.
    """
    _require_cuda(q, k_cache, v_cache, indices, weights)
    d = q.shape[-1]
    q5 = _inner_contiguous(q)
    kc5 = _as_cache5(k_cache, d)
    vc5 = _as_cache5(v_cache, d)
    _check_shapes(q5, kc5, vc5, indices, weights)
    idx32 = indices.to(torch.int32).contiguous()
    w32 = weights.to(torch.float32).contiguous()
    obo = (float(sm_n) if sm_n else 1.0) if softmax_off_by_one else 0.0
    return _GcaIndexed.apply(q5, kc5, vc5, idx32, w32, float(sm_scale), obo, int(algo), bool(token_major_out))


def _pregathered_views(q, k, v, weights):
    if q.dim() != 4 or k.dim() != 5 or v.dim() != 5:
        raise ValueError("expected q (Z,Hq,S,D), k/v (Z,Hkv,K,L,D)")
    if weights.dim() != 2:
        raise ValueError("weights must be 2-D (Z, K)")          # ltriton/gca.py:699
    if q.shape[-1] != k.shape[-1] or k.shape != v.shape:
        raise ValueError("head dims / k,v shapes differ")       # ltriton/gca.py:697
    z, kk = k.shape[0], k.shape[2]
    q5 = _inner_contiguous(q).unsqueeze(1)                       # (Z, 1, Hq, S, D)
    kc5 = _inner_contiguous(k).permute(0, 2, 3, 1, 4)            # (Z, K, L, Hkv, D) view
    vc5 = _inner_contiguous(v).permute(0, 2, 3, 1, 4)
    idx32 = torch.arange(kk, dtype=torch.int32, device=q.device).view(1, 1, kk).expand(z, 1, kk).contiguous()
    w32 = weights.to(torch.float32).reshape(z, 1, kk).contiguous()
    return q5, kc5, vc5, idx32, w32


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, weights: torch.Tensor,
              sm_scale: float, sm_n: float = 0.0) -> torch.Tensor:
    """Drop-in for ``ltriton.gca.attention`` (``_attention.apply``, ``ltriton/gca.py:681-844``).

    q (Z, Hq, S, D); k, v (Z, Hkv, K, L, D) pre-gathered chunks; weights (Z, K).
    Differentiable in q, k, v and weights; ``sm_n`` is inert as in the reference kernel
    (its ``l_i = sm_n`` start value is multiplied by zero in the first softmax step,
    ``ltriton/gca.py:48-49,187``).
    """
    _require_cuda(q, k, v, weights)
    q5, kc5, vc5, idx32, w32 = _pregathered_views(q, k, v, weights)
    out = _GcaIndexed.apply(q5, kc5, vc5, idx32, w32, float(sm_scale), 0.0, ALGO_AUTO)
    return out.squeeze(1)


def _forward_nograd(q5, kc5, vc5, idx32, w32, sm_scale, off_by_one, algo) -> torch.Tensor:
    n, j, hq, s, d = q5.shape
    out = torch.empty((n, j, hq, s, d), dtype=q5.dtype, device=q5.device)
    with torch.cuda.device(q5.device):
        a = _fwd_args(q5, kc5, vc5, idx32, w32, out, None, sm_scale, off_by_one, algo)
        if s <= 16:
            _lib.call("gca_decode", C.byref(a), _stream())
        else:
            if s != 64 and algo == ALGO_AUTO:
                a.algo = ALGO_SIMT
            _lib.call("gca_fwd", C.byref(a), _stream())
    _maybe_check(q5.device)
    return out


@torch.no_grad()
def gca_kv_cache(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, weights: torch.Tensor,
                 sm_scale: float, sm_n: float = 0.0) -> torch.Tensor:
    """Drop-in for ``ltriton.gca.gca_kv_cache`` (``ltriton/gca.py:846-888``): no autograd;
    q (Z, Hq, Sq, D) with Sq = 1 or 2 while decoding and Sq = 64 for eval prefill
    (``model/DRT.py:379-382``)."""
    _require_cuda(q, k, v, weights)
    q5, kc5, vc5, idx32, w32 = _pregathered_views(q, k, v, weights)
    return _forward_nograd(q5, kc5, vc5, idx32, w32, float(sm_scale), 0.0, ALGO_AUTO).squeeze(1)


@torch.no_grad()
def gca_indexed_nograd(q, k_cache, v_cache, indices, weights, sm_scale, sm_n: float = 0.0, *,
                       softmax_off_by_one: bool = False, algo: int = ALGO_AUTO) -> torch.Tensor:
    """Inference form of ``gca_indexed`` for any Sq in [1, 64] (decode uses 1 or 2 rows)."""
    _require_cuda(q, k_cache, v_cache, indices, weights)
    d = q.shape[-1]
    q5 = _inner_contiguous(q)
    kc5 = _as_cache5(k_cache, d)
    vc5 = _as_cache5(v_cache, d)
    _check_shapes(q5, kc5, vc5, indices, weights)
    idx32 = indices.to(torch.int32).contiguous()
    w32 = weights.to(torch.float32).contiguous()
    obo = (float(sm_n) if sm_n else 1.0) if softmax_off_by_one else 0.0
    return _forward_nograd(q5, kc5, vc5, idx32, w32, float(sm_scale), obo, int(algo))


def gca_forward_with_lse(q, k_cache, v_cache, indices, weights, sm_scale, *, off_by_one: float = 0.0,
                         algo: int = ALGO_AUTO) -> Tuple[torch.Tensor, torch.Tensor]:
    """Forward returning (out, lse) with lse (N*J, Hq, K, S) in base 2 -- for tests and tools."""
    d = q.shape[-1]
    q5, kc5, vc5 = _inner_contiguous(q), _as_cache5(k_cache, d), _as_cache5(v_cache, d)
    _check_shapes(q5, kc5, vc5, indices, weights)
    idx32 = indices.to(torch.int32).contiguous()
    w32 = weights.to(torch.float32).contiguous()
    n, j, hq, s, _ = q5.shape
    out = torch.empty((n, j, hq, s, d), dtype=q5.dtype, device=q5.device)
    lse = torch.empty((n * j, hq, idx32.shape[-1], s), dtype=torch.float32, device=q5.device)
    with torch.cuda.device(q5.device):
        a = _fwd_args(q5, kc5, vc5, idx32, w32, out, lse, sm_scale, off_by_one, algo)
        _lib.call("gca_fwd", C.byref(a), _stream())
    return out, lse
