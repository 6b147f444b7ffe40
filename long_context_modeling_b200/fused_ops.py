"""The projections either side of GCA as tensor-core GEMMs with fused prologue / epilogue work
(inference: no autograd): pre-norm RMSNorm + ``q_proj`` (``model/DRT.py:352-355``) and ``o_proj`` +
residual add (``model/DRT.py:385`` and the decoder layer's ``residual + hidden_states``, ``:484``).

``RMSNorm(x) W^T = diag(1 / rms(x)) . x . (W diag(g))^T``: the norm's gain ``g`` is folded into the
weight's columns once, the GEMM reads the raw activations, and its epilogue scales each output row
by ``1 / rms`` -- the normalised activations are never written or re-read.  The reference gets the
same effect from third-party fused kernels (flash-attn's RMSNorm, xformers); here it is the
library's own tcgen05 GEMM (``gca_linear``) plus a one-pass row reduction (``gca_row_rms``).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from .gca import _status, _stream


def _rows(t: torch.Tensor) -> torch.Tensor:
    """(..., D) -> a 2-D view (M, D) with one row stride; copies only if no such view exists."""
    if t.dim() == 2 and t.stride(1) == 1:
        return t
    if t.is_contiguous():
        return t.view(-1, t.shape[-1])
    return t.reshape(-1, t.shape[-1]).contiguous()


def _require(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name}: the fused projections run on a CUDA device only (no CPU fallback)")
    if t.dtype != torch.bfloat16:
        raise ValueError(f"{name}: expected bfloat16, got {t.dtype}")


def row_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """1 / sqrt(mean(x^2, -1) + eps) per row of x (..., D) bf16 -> float32 (M,)."""
    _require(x, "row_rms")
    x2 = _rows(x)
    out = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
    a = _lib.RowRmsArgs()
    a.x, a.row_scale, a.M, a.x_stride, a.D, a.eps = x2.data_ptr(), out.data_ptr(), x2.shape[0], x2.stride(0), x2.shape[1], eps
    _lib.call("gca_row_rms", C.byref(a), _stream())
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, row_scale: Optional[torch.Tensor] = None,
           residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[m] = row_scale[m] * (x[m] @ weight.T) + residual[m]; x (..., K), weight (N, K), bf16."""
    _require(x, "linear")
    _require(weight, "linear weight")
    x2, n = _rows(x), weight.shape[0]
    shape = x.shape[:-1] + (n,)
    if out is None:
        out = torch.empty(shape, dtype=torch.bfloat16, device=x.device)
    o2 = _rows(out)
    if o2.data_ptr() != out.data_ptr():
        raise ValueError("linear: `out` must be viewable as (M, N) rows")
    a = _lib.LinearArgs()
    a.x, a.w, a.out = x2.data_ptr(), weight.data_ptr(), o2.data_ptr()
    a.M, a.N, a.K = x2.shape[0], n, x2.shape[1]
    a.x_stride, a.w_stride, a.out_stride = x2.stride(0), weight.stride(0), o2.stride(0)
    if residual is not None:
        _require(residual, "linear residual")
        r2 = _rows(residual)
        if r2.shape != o2.shape:
            raise ValueError(f"linear: residual {tuple(residual.shape)} does not match the output {tuple(shape)}")
        a.residual, a.residual_stride = r2.data_ptr(), r2.stride(0)
    if row_scale is not None:
        if row_scale.dtype != torch.float32 or row_scale.numel() != x2.shape[0] or not row_scale.is_contiguous():
            raise ValueError("linear: row_scale must be contiguous float32 with one value per row")
        a.row_scale = row_scale.data_ptr()
    a.status = _status(x.device).data_ptr()
    _lib.call("gca_linear", C.byref(a), _stream())
    return out


def fold_gain(weight: torch.Tensor, gain: torch.Tensor) -> torch.Tensor:
    """W diag(g) as bf16: the projection weight with the preceding RMSNorm's gain folded in."""
    return (weight.float() * gain.float()[None, :]).to(torch.bfloat16).contiguous()


def rmsnorm_linear(x: torch.Tensor, folded_weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm(x) @ W.T with ``folded_weight = fold_gain(W, norm.weight)``: one row reduction over x
    and one GEMM over the raw x whose epilogue applies 1 / rms."""
    return linear(x, folded_weight, row_scale=row_rms(x, eps))


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate_up[..., :I]) * gate_up[..., I:] for the output (..., 2 I) of one stacked gate|up projection
    (the reference's fused SwiGLU activation, ``model/llama.py:290-300``): one launch, one rounding."""
    _require(gate_up, "silu_mul")
    x2 = _rows(gate_up)
    inter = x2.shape[1] // 2
    if x2.shape[1] != 2 * inter:
        raise ValueError("silu_mul: the last dimension must hold gate and up halves of equal width")
    out = torch.empty((x2.shape[0], inter), dtype=torch.bfloat16, device=gate_up.device)
    _lib.call("gca_silu_mul", x2.data_ptr(), out.data_ptr(), x2.shape[0], inter, x2.stride(0), out.stride(0), _stream())
    return out.view(*gate_up.shape[:-1], inter)


def window_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int, slopes: Optional[torch.Tensor] = None,
                  sm_scale: Optional[float] = None) -> torch.Tensor:
    """Sliding-window causal attention with ALiBi for a few new positions against the cached window
    (``flash_attn_with_kvcache(..., causal=True, window_size=(window, 0), alibi_slopes=slopes)``,
    ``model/llama.py:684-688``).  q (N, Hq, Sq, 64), k / v (N, Hkv, T, 64) bf16 -- any strides with the
    head dimension contiguous; the query rows stand at positions T - Sq .. T - 1.  Returns (N, Hq, Sq, 64)."""
    a = _lib.WindowDecodeArgs()
    out = _fill_window_args(a, q, k, v, window, slopes, sm_scale)
    _lib.call("gca_window_decode", C.byref(a), _stream())
    return out


def _fill_window_args(a, q, k, v, window, slopes, sm_scale) -> torch.Tensor:
    for t, name in ((q, "q"), (k, "k"), (v, "v")):
        _require(t, f"window_decode {name}")
        if t.dim() != 4 or t.shape[-1] != 64 or t.stride(-1) != 1:
            raise ValueError(f"window_decode: {name} must be (N, H, L, 64) with contiguous head dimension")
    n, hq, sq, _ = q.shape
    hkv, t_len = k.shape[1], k.shape[2]
    out = torch.empty((n, hq, sq, 64), dtype=torch.bfloat16, device=q.device)
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    if slopes is not None:
        if slopes.dtype != torch.float32 or slopes.numel() != hq or not slopes.is_contiguous() or not slopes.is_cuda:
            raise ValueError("window_decode: slopes must be contiguous float32 (Hq,) on the device")
        a.alibi_slopes = slopes.data_ptr()
    for i in range(3):
        a.q_stride[i], a.o_stride[i], a.k_stride[i], a.v_stride[i] = q.stride(i), out.stride(i), k.stride(i), v.stride(i)
    a.N, a.Hq, a.Hkv, a.Sq, a.T, a.window = n, hq, hkv, sq, t_len, int(window)
    a.sm_scale = float(sm_scale) if sm_scale is not None else 0.125
    return out


def window_ring_decode(q: torch.Tensor, k_ring: torch.Tensor, v_ring: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
                       rows_written: torch.Tensor, window: int, slopes: Optional[torch.Tensor] = None,
                       sm_scale: Optional[float] = None) -> torch.Tensor:
    """``window_decode`` for one new position per sequence with the append folded in and the window
    kept as a RING that never moves: ``k_ring`` / ``v_ring`` (N, Hkv, T, 64) hold the last T positions,
    the oldest at row ``rows_written mod T``; ``k_new`` / ``v_new`` (N, Hkv, 1, 64) or (N, Hkv, 64) are
    attended to as the newest position and stored over the oldest row.  ``rows_written`` is a device int64
    scalar the CALLER advances by one after the step (all layers of a model share one counter), so that a
    captured CUDA graph can replay the step; it must stay below 2^32 (subtract a multiple of T long before).
    q (N, Hq, 1, 64).  ``torch.roll(ring, -(rows_written % T), 2)``
    gives the window back in order."""
    for t, name in ((k_new, "k_new"), (v_new, "v_new")):
        _require(t, f"window_ring_decode {name}")
    if not rows_written.is_cuda:
        raise RuntimeError("window_ring_decode rows_written: the fused projections run on a CUDA device only (no CPU fallback)")
    if rows_written.dtype != torch.int64 or rows_written.numel() != 1:
        raise ValueError("window_ring_decode: rows_written must be one int64 on the device")
    n, hkv = k_ring.shape[0], k_ring.shape[1]
    kn, vn = k_new.reshape(n, hkv, 64) if k_new.dim() == 4 else k_new, v_new.reshape(n, hkv, 64) if v_new.dim() == 4 else v_new
    if kn.stride(2) != 1 or vn.stride(2) != 1 or kn.stride()[:2] != vn.stride()[:2]:
        raise ValueError("window_ring_decode: new rows must be bf16 with a contiguous head dimension and equal strides")
    a = _lib.WindowRingDecodeArgs()
    out = _fill_window_args(a.attn, q, k_ring, v_ring, window, slopes, sm_scale)
    a.k_new, a.v_new, a.rows_written = kn.data_ptr(), vn.data_ptr(), rows_written.data_ptr()
    a.new_stride[0], a.new_stride[1] = kn.stride(0), kn.stride(1)
    _lib.call("gca_window_ring_decode", C.byref(a), _stream())
    return out


def linear_cross_entropy(x: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor,
                         row_scale: Optional[torch.Tensor] = None, return_lse: bool = False):
    """Per-row cross-entropy of ``x @ weight.T`` against ``targets`` without materialising the logits
    (``lm_head`` + ``CrossEntropyLoss(ignore_index=-100, reduction='none')``, ``model/DRT.py:1055-1064``;
    forward only).  x (..., K) bf16, weight (V, K) bf16, targets (...) int64 with negative = ignored.
    Returns float32 losses shaped like ``targets`` (and the natural-log logsumexp when asked)."""
    _require(x, "linear_cross_entropy")
    _require(weight, "linear_cross_entropy weight")
    x2 = _rows(x)
    t = targets.reshape(-1).to(torch.int64).contiguous()
    if t.numel() != x2.shape[0] or not t.is_cuda:
        raise ValueError("linear_cross_entropy: one int64 target per row, on the device")
    m, v = x2.shape[0], weight.shape[0]
    loss = torch.empty(m, dtype=torch.float32, device=x.device)
    lse = torch.empty(m, dtype=torch.float32, device=x.device) if return_lse else None
    lib = _lib.lib()
    nbytes = lib.gca_linear_ce_workspace_bytes(m, v)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
    a = _lib.LinearCeArgs()
    a.x, a.w, a.targets, a.loss = x2.data_ptr(), weight.data_ptr(), t.data_ptr(), loss.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
    a.M, a.N, a.K, a.x_stride, a.w_stride = m, v, x2.shape[1], x2.stride(0), weight.stride(0)
    if row_scale is not None:
        if row_scale.dtype != torch.float32 or row_scale.numel() != m or not row_scale.is_contiguous():
            raise ValueError("linear_cross_entropy: row_scale must be contiguous float32 with one value per row")
        a.row_scale = row_scale.data_ptr()
    a.status = _status(x.device).data_ptr()
    _lib.call("gca_linear_cross_entropy", C.byref(a), _stream())
    loss = loss.view(targets.shape)
    return (loss, lse.view(targets.shape)) if return_lse else loss


def window_shift_append(k_window: torch.Tensor, v_window: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor) -> None:
    """Move a full cached window on by one position IN PLACE: every (n, head) block of ``k_window`` /
    ``v_window`` (N, H, T, 64; the T x 64 block contiguous) drops its oldest row and takes the row of
    ``k_new`` / ``v_new`` (N, H, 1, 64) or (N, H, 64) at the end -- the reference's ``torch.cat`` + slice of
    its KV cache without a second buffer."""
    for t, name in ((k_window, "k_window"), (v_window, "v_window"), (k_new, "k_new"), (v_new, "v_new")):
        _require(t, f"window_shift_append {name}")
    n, h, t_len, d = k_window.shape
    if d != 64 or v_window.shape != k_window.shape or k_window.stride(3) != 1 or k_window.stride(2) != 64 or \
            v_window.stride(3) != 1 or v_window.stride(2) != 64 or v_window.stride()[:2] != k_window.stride()[:2]:
        raise ValueError("window_shift_append: windows must be (N, H, T, 64) with contiguous (T, 64) blocks and equal strides")
    kn, vn = k_new.reshape(n, h, 64) if k_new.dim() == 4 else k_new, v_new.reshape(n, h, 64) if v_new.dim() == 4 else v_new
    if kn.stride(2) != 1 or vn.stride(2) != 1 or kn.stride()[:2] != vn.stride()[:2]:
        raise ValueError("window_shift_append: new rows must have a contiguous head dimension and equal strides")
    a = _lib.WindowAppendArgs()
    a.k_window, a.v_window, a.k_new, a.v_new = k_window.data_ptr(), v_window.data_ptr(), kn.data_ptr(), vn.data_ptr()
    a.window_stride[0], a.window_stride[1] = k_window.stride(0), k_window.stride(1)
    a.new_stride[0], a.new_stride[1] = kn.stride(0), kn.stride(1)
    a.N, a.H, a.T = n, h, t_len
    _lib.call("gca_window_shift_append", C.byref(a), _stream())
