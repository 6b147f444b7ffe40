"""The GCA sub-layer as an ``nn.Module``: mirror of ``TritonGroupCrossAttention``
(``model/DRT.py:304-398``) with the same parameter names (``pre_norm``, ``q_proj``,
``o_proj``) so reference checkpoints load; and of ``GroupCrossAttention``
(``model/DRT.py:235-302``), the variant the reference runs through flash-attn when
``_triton_gca`` is off, on the same kernels.

``forward`` keeps the reference's argument meaning (pre-gathered chunks).  ``forward_indexed``
is the fast path: the query is handed to the kernel as a strided view of the projection
output and K/V are read from the chunk cache by retrieved index, so neither the gather
(``model/DRT.py:198-199``) nor the two layout copies (``:328-332``, ``:372-378``) happen.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from . import fused_ops, gca


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        dt = x.dtype
        x = x.float()
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps)
        return (x * self.weight.float()).to(dt)


def preprocess_chunk_kv_cache(chunk_k: torch.Tensor, chunk_v: torch.Tensor, weights: torch.Tensor, num_heads: int):
    """``TritonGroupCrossAttention.preprocess_chunk_kv_cache`` (``model/DRT.py:320-332``):
    chunk_k/v (N, D*K, S, h*d), weights (N, D, K) -> k, v (N*D, h, K, S, d), weights (N*D, K)."""
    n, dk, s, hd = chunk_k.shape
    kk = weights.shape[-1]
    d = dk // kk
    hdim = hd // num_heads

    def split(t):
        return t.reshape(n, d, kk, s, num_heads, hdim).permute(0, 1, 4, 2, 3, 5).reshape(n * d, num_heads, kk, s, hdim).contiguous()

    return split(chunk_k), split(chunk_v), weights.reshape(n * d, kk)


class TritonGroupCrossAttention(nn.Module):
    """``TritonGroupCrossAttention(config)`` like the reference's constructor
    (``model/DRT.py:305-318``: reads ``hidden_size``, ``num_attention_heads``, ``enc_chunk_size``,
    ``chunk_topk``, ``rms_norm_eps``, ``attention_bias``, ``enable_softmax_one``), or the same
    values spelled out: ``TritonGroupCrossAttention(hidden_size, num_heads, ...)``."""

    def __init__(self, hidden_size, num_heads: int = None, enc_chunk_size: int = 63, chunk_topk: int = 8,
                 rms_norm_eps: float = 1e-5, attention_bias: bool = False, enable_softmax_one: bool = False):
        super().__init__()
        if hasattr(hidden_size, "hidden_size"):              # a model config object
            config = hidden_size
            hidden_size, num_heads = config.hidden_size, config.num_attention_heads
            enc_chunk_size = getattr(config, "enc_chunk_size", enc_chunk_size)
            chunk_topk = getattr(config, "chunk_topk", chunk_topk)
            rms_norm_eps = getattr(config, "rms_norm_eps", rms_norm_eps)
            attention_bias = getattr(config, "attention_bias", attention_bias)
            enable_softmax_one = getattr(config, "enable_softmax_one", enable_softmax_one)
        if num_heads is None:
            raise TypeError("TritonGroupCrossAttention needs a config object or (hidden_size, num_heads, ...)")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.head_dim = hidden_size // num_heads
        self.enc_chunk_size = enc_chunk_size
        self.topK = chunk_topk
        self.pre_norm = RMSNorm(hidden_size, eps=rms_norm_eps)
        self.q_proj = nn.Linear(hidden_size, num_heads * self.head_dim, bias=attention_bias)
        self.o_proj = nn.Linear(hidden_size, num_heads * self.head_dim, bias=attention_bias)
        self.enable_softmax_one = enable_softmax_one
        self.sm_n = 1.0 if enable_softmax_one else 0.0          # model/DRT.py:317-318

    @classmethod
    def from_config(cls, config):
        return cls(config)

    preprocess_chunk_kv_cache = staticmethod(preprocess_chunk_kv_cache)

    def _zeros(self, hidden_states):
        return torch.zeros((hidden_states.shape[0], hidden_states.shape[1] * hidden_states.shape[2],
                            hidden_states.shape[-1]), dtype=hidden_states.dtype, device=hidden_states.device)

    def _pad_first_chunk(self, hidden_states, o):
        """The first chunk has nothing to retrieve: its rows are zeros (model/DRT.py:387-394)."""
        ret = torch.zeros((hidden_states.shape[0], hidden_states.shape[1] * hidden_states.shape[2],
                           hidden_states.shape[-1]), dtype=o.dtype, device=o.device)
        ret[:, -o.shape[1]:, :] = o
        return ret

    def forward(self, hidden_states: torch.Tensor, chunk_k: torch.Tensor, chunk_v: torch.Tensor,
                weights: torch.Tensor) -> torch.Tensor:
        """hidden_states (N, D, S, dim); chunk_k/v (N*D', h, K, S, d); weights (N*D', K) with
        D' = D-1 when D > 1 (the first chunk is skipped) -- ``model/DRT.py:345-398``."""
        hs = self.pre_norm(hidden_states)
        chunk_size = hs.shape[1]
        q = self.q_proj(hs)
        n, dd, s, _ = q.shape
        q = q.view(n, dd, s, self.num_heads, self.head_dim).permute(0, 1, 3, 2, 4)   # N D h S d (view)
        if weights.shape[0] * weights.shape[1] == 0:
            return self._zeros(hidden_states)
        if chunk_size > 1:
            q = q[:, 1:]
        q = q.reshape(-1, self.num_heads, s, self.head_dim).contiguous()
        scale = 1.0 / math.sqrt(self.head_dim)
        if chunk_size > 1 and self.training:
            vals = gca.attention(q, chunk_k, chunk_v, weights, scale, self.sm_n)
        else:
            vals = gca.gca_kv_cache(q, chunk_k, chunk_v, weights, scale, self.sm_n)
        vals = vals.view(n, -1, self.num_heads, s, self.head_dim).permute(0, 1, 3, 2, 4).reshape(n, -1, self.hidden_size)
        o = self.o_proj(vals)
        return self._pad_first_chunk(hidden_states, o) if chunk_size > 1 else o

    def _folded_q_weight(self) -> torch.Tensor:
        """q_proj.weight with pre_norm's gain folded in, cached until either parameter changes."""
        key = (self.q_proj.weight._version, self.pre_norm.weight._version, self.q_proj.weight.data_ptr())
        if getattr(self, "_folded_key", None) != key:
            self._folded_w = fused_ops.fold_gain(self.q_proj.weight.detach(), self.pre_norm.weight.detach())
            self._folded_key = key
        return self._folded_w

    def forward_fused(self, hidden_states: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      indices: torch.Tensor, weights: torch.Tensor, residual: torch.Tensor = None,
                      first_chunk_retrieves: bool = False) -> torch.Tensor:
        """Inference form of ``forward_indexed`` (bf16, no autograd, no projection bias) with the small
        operations fused into the two projections: RMSNorm's row scale is the q_proj GEMM's epilogue
        (gain folded into the weight), and ``residual`` -- the decoder layer's ``residual +
        gca(...)`` (``model/DRT.py:484``), shape (N, D*S, dim) -- is added by the o_proj GEMM's
        epilogue.  Rows of a skipped first chunk come back as the residual alone (zeros without one),
        as in ``model/DRT.py:387-394``."""
        if self.q_proj.bias is not None or self.o_proj.bias is not None:
            raise ValueError("forward_fused: projection biases are not supported")
        n, dd, s, dim = hidden_states.shape
        q = fused_ops.rmsnorm_linear(hidden_states, self._folded_q_weight(), self.pre_norm.eps)
        skip_first = dd > 1 and not first_chunk_retrieves
        out = torch.empty((n, dd * s, dim), dtype=torch.bfloat16, device=hidden_states.device)
        if skip_first or indices.shape[1] * indices.shape[2] == 0:
            lead = s if indices.shape[1] * indices.shape[2] else dd * s
            if residual is None:
                out[:, :lead].zero_()
            else:
                out[:, :lead] = residual[:, :lead]
            if lead == dd * s:
                return out
        q5 = q.view(n, dd, s, self.num_heads, self.head_dim).permute(0, 1, 3, 2, 4)
        if skip_first:
            q5 = q5[:, 1:]
        vals = gca.gca_indexed_nograd(q5, k_cache, v_cache, indices, weights, 1.0 / math.sqrt(self.head_dim), self.sm_n)
        vals = vals.permute(0, 1, 3, 2, 4).reshape(n, -1, self.hidden_size)
        first = s if skip_first else 0
        w = self.o_proj.weight.detach()
        if first == 0:                           # no skipped chunk: all rows share one row stride, one GEMM
            fused_ops.linear(vals, w, residual=residual, out=out)
            return out
        for b in range(n):                       # one GEMM per sequence: a sequence's rows share one row stride
            fused_ops.linear(vals[b], w, residual=None if residual is None else residual[b, first:], out=out[b, first:])
        return out

    def forward_indexed(self, hidden_states: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                        indices: torch.Tensor, weights: torch.Tensor, first_chunk_retrieves: bool = False) -> torch.Tensor:
        """hidden_states (N, D, S, dim); caches (N, C, L, h*d); indices / weights (N, D', K)
        where D' = D-1 for D > 1 (query chunk j uses the retrieval made by chunk j-1) and
        D' = D = 1 while decoding.  ``first_chunk_retrieves``: the chunks are a later SEGMENT of a
        long prompt whose first chunk uses the retrieval made at the end of the previous segment:
        D' = D and no chunk is skipped."""
        hs = self.pre_norm(hidden_states)
        chunk_size = hs.shape[1]
        q = self.q_proj(hs)
        n, dd, s, _ = q.shape
        if indices.shape[1] * indices.shape[2] == 0:
            return self._zeros(hidden_states)
        q5 = q.view(n, dd, s, self.num_heads, self.head_dim).permute(0, 1, 3, 2, 4)  # strided view, no copy
        skip_first = chunk_size > 1 and not first_chunk_retrieves
        if skip_first:
            q5 = q5[:, 1:]
        scale = 1.0 / math.sqrt(self.head_dim)
        if torch.is_grad_enabled() and (q5.requires_grad or k_cache.requires_grad or weights.requires_grad):
            vals = gca.gca_indexed(q5, k_cache, v_cache, indices, weights, scale, self.sm_n, token_major_out=True)
        else:
            vals = gca.gca_indexed_nograd(q5, k_cache, v_cache, indices, weights, scale, self.sm_n)
        vals = vals.permute(0, 1, 3, 2, 4).reshape(n, -1, self.hidden_size)
        o = self.o_proj(vals)
        return self._pad_first_chunk(hidden_states, o) if skip_first else o


class GroupCrossAttention(TritonGroupCrossAttention):
    """Mirror of the reference's non-Triton ``GroupCrossAttention`` (``model/DRT.py:235-302``):
    same parameters, but the retrieved chunks arrive as (N*D'*K, S, h, d) -- the layout
    ``flash_attn_func`` wants -- and ``sm_n`` does not exist.  The reference expands the query
    K-fold, runs K independent attentions and merges them with an einsum; here the same tensors
    are handed to the GCA kernels as strided views (no expansion, no copy)."""

    def __init__(self, hidden_size, num_heads: int = None, enc_chunk_size: int = 63, chunk_topk: int = 8,
                 rms_norm_eps: float = 1e-5, attention_bias: bool = False):
        super().__init__(hidden_size, num_heads, enc_chunk_size, chunk_topk, rms_norm_eps, attention_bias, False)
        self.enable_softmax_one, self.sm_n = False, 0.0        # this variant has no sm_n (model/DRT.py:235-302)

    @staticmethod
    def preprocess_chunk_kv_cache(chunk_k: torch.Tensor, chunk_v: torch.Tensor, weights: torch.Tensor, num_heads: int):
        """``model/DRT.py:247-256``: chunk_k/v (N, D*K, S, h*d) -> (N*D*K, S, h, d) views; weights unchanged."""
        n, dk, s, hd = chunk_k.shape
        return (chunk_k.reshape(n * dk, s, num_heads, hd // num_heads),
                chunk_v.reshape(n * dk, s, num_heads, hd // num_heads), weights)

    def forward(self, hidden_states: torch.Tensor, chunk_k: torch.Tensor, chunk_v: torch.Tensor,
                weights: torch.Tensor) -> torch.Tensor:
        """hidden_states (N, D, S, dim); chunk_k/v (N*D'*K, S, h, d); weights (N, D', K)."""
        if weights.shape[1] * weights.shape[2] == 0:
            return self._zeros(hidden_states)
        n, dprime, kk = weights.shape
        s, h, d = chunk_k.shape[1:]
        k5 = chunk_k.view(n * dprime, kk, s, h, d).permute(0, 3, 1, 2, 4)      # (Z, h, K, S, d) view
        v5 = chunk_v.view(n * dprime, kk, s, h, d).permute(0, 3, 1, 2, 4)
        return super().forward(hidden_states, k5, v5, weights.reshape(n * dprime, kk))
