"""A minimal DRT model body around the GCA / retrieval hot path.

This is NOT a port of the reference's ``model/DRT.py`` + ``model/llama.py`` (1,900 lines of
HuggingFace-derived plumbing): it restates, in ~400 lines of plain PyTorch, just enough of the
architecture to DRIVE the hot path the way the reference model drives it, so that the two
whole-model legs of the headline metric (one DRT-16K training step, greedy generation with a
long chunk cache) can be measured with this repository's kernels plugged in, and so that the
reference's one behavioural pin of the decode path -- incremental decoding gives the argmax of
a teacher-forced forward (``tests/generation_unittest.py:16-37``) -- can be tested.

What follows the reference (paths inside the reference project):

* chunking: a landmark id is appended after every ``enc_chunk_size`` = 63 tokens, 64 positions
  per chunk (``model/DRT.py:954-961``); logits at landmark positions are dropped.
* lower stack: pre-norm decoder layers, causal self-attention with a sliding window of
  ``slide_window`` positions and ALiBi slopes ``2^(-8 (h+1) / H)``, no rotary embedding
  (``model/llama.py:315-319,661-689``); SwiGLU MLP (``llama.py:278-300``).
* chunk encoder: ``enc_prenorm`` -> bidirectional layers with rotary embedding over each
  64-position chunk -> final norm; landmark embedding = last position; K/V = two linear maps
  of the encoder output with the landmark row zeroed (``model/DRT.py:758-784``).
* retrieval per group: query landmark = ``lmk_norms[g]`` of the hidden state at the landmark
  positions; top-k over earlier chunks; query chunk j uses the retrieval made by chunk j-1
  (``model/DRT.py:819-824,609-641``).
* upper layers: ``x = x + SelfAttn(LN(x)); r = x; g = GCA(x); y = LN2(r + g); out = r + MLP(y)``
  -- the GCA output feeds the MLP only (``model/DRT.py:457-491``).
* decoding: hidden states of the lower stack are staged until a chunk is complete, then encoded
  and appended; at a chunk boundary the step carries two positions (token, landmark) and the
  retrieval for the NEXT chunk is made after the current step's GCA has fetched its chunks
  (``model/DRT.py:787-849``).

Deliberate differences: the decode-time retrieval applies ``lmk_norms[g]`` like the batch path
(the reference skips it there, ``model/DRT.py:837``, which changes weights but not the ranking
under freshly initialised norms); dense projections, norms and the windowed self-attention are
plain torch ops (cuBLAS / SDPA): they are callers of the hot path, not part of it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .chunk_cache import ChunkKVManager
from .modules import RMSNorm, TritonGroupCrossAttention
from .retrieval import lmk_score_topk, retrieve


@dataclass
class DRTConfig:
    hidden_size: int = 768
    num_attention_heads: int = 12
    intermediate_size: int = 2048
    vocab_size: int = 50265
    decoder_layers: List[int] = field(default_factory=lambda: [6, 6])     # [lower, group 0, group 1, ...]
    encoder_layers: int = 2
    enc_chunk_size: int = 63
    chunk_topk: int = 8
    slide_window: int = 512
    rms_norm_eps: float = 1e-5
    attention_bias: bool = False
    enable_softmax_one: bool = False
    initializer_range: float = 0.02
    chunk_id: int = 50264                 # the landmark token

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


def alibi_slopes(heads: int) -> torch.Tensor:
    """``1 / x^(i+1)`` with ``x = (2^8)^(1/H)`` (``model/llama.py:315-319``)."""
    return torch.tensor([2.0 ** (-8.0 * (i + 1) / heads) for i in range(heads)])


def windowed_alibi_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int, slopes: torch.Tensor) -> torch.Tensor:
    """Causal self-attention where query i sees keys i - window .. i, with ALiBi bias
    ``-slope_h (i - j)``.  q, k, v (N, H, L, d).  Computed block-banded: queries in blocks of
    ``window`` positions attend to their own and the previous block (never a dense L x L mask)."""
    n, h, l, d = q.shape
    b = window
    pad = (-l) % b
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, pad)) for t in (q, k, v))
    nb = (l + pad) // b
    qb, kb, vb = (t.view(n, h, nb, b, d) for t in (q, k, v))
    i = torch.arange(b, device=q.device).view(b, 1)
    j = torch.arange(2 * b, device=q.device).view(1, 2 * b) - b          # key position relative to the block start
    dist = (i - j).float()                                                # >= 0 for visible keys
    bias = -slopes.to(q.device).view(h, 1, 1).float() * dist
    bias = bias.masked_fill((dist < 0) | (dist > window), float("-inf")).to(q.dtype)       # (H, b, 2b)
    outs = []
    # block 0 has no previous block
    outs.append(F.scaled_dot_product_attention(qb[:, :, :1], kb[:, :, :1], vb[:, :, :1], attn_mask=bias[:, :, b:].view(1, h, 1, b, b)))
    if nb > 1:
        k2 = torch.cat([kb[:, :, :-1], kb[:, :, 1:]], dim=3)
        v2 = torch.cat([vb[:, :, :-1], vb[:, :, 1:]], dim=3)
        outs.append(F.scaled_dot_product_attention(qb[:, :, 1:], k2, v2, attn_mask=bias.view(1, h, 1, b, 2 * b)))
    out = torch.cat(outs, dim=2).reshape(n, h, nb * b, d)
    return out[:, :, :l]


def rotary(x: torch.Tensor, base: float = 10000.0) -> torch.Tensor:
    """Rotary position embedding over the second-to-last axis (positions 0 .. S-1); x (..., S, d)."""
    s, d = x.shape[-2], x.shape[-1]
    inv = 1.0 / (base ** (torch.arange(0, d, 2, device=x.device).float() / d))
    ang = torch.arange(s, device=x.device).float().view(s, 1) * inv.view(1, -1)
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1).to(x.dtype), torch.cat([ang.sin(), ang.sin()], -1).to(x.dtype)
    x1, x2 = x[..., : d // 2], x[..., d // 2:]
    return x * cos + torch.cat([-x2, x1], -1) * sin


class MLP(nn.Module):
    def __init__(self, cfg: DRTConfig):
        super().__init__()
        self.gate_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.up_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.down_proj = nn.Linear(cfg.intermediate_size, cfg.hidden_size, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class SelfAttention(nn.Module):
    """Decoder form: causal, sliding window, ALiBi, optional KV cache.  Encoder form
    (``bidirectional=True``): full attention inside a chunk with rotary embedding."""

    def __init__(self, cfg: DRTConfig, bidirectional: bool = False):
        super().__init__()
        self.h, self.d, self.window, self.bidirectional = cfg.num_attention_heads, cfg.head_dim, cfg.slide_window, bidirectional
        self.q_proj = nn.Linear(cfg.hidden_size, cfg.hidden_size, bias=cfg.attention_bias)
        self.k_proj = nn.Linear(cfg.hidden_size, cfg.hidden_size, bias=cfg.attention_bias)
        self.v_proj = nn.Linear(cfg.hidden_size, cfg.hidden_size, bias=cfg.attention_bias)
        self.o_proj = nn.Linear(cfg.hidden_size, cfg.hidden_size, bias=cfg.attention_bias)
        self.register_buffer("slopes", alibi_slopes(self.h), persistent=False)

    def forward(self, x: torch.Tensor, cache: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, use_cache: bool = False):
        n, l, _ = x.shape
        q, k, v = (p(x).view(n, l, self.h, self.d).transpose(1, 2) for p in (self.q_proj, self.k_proj, self.v_proj))
        if self.bidirectional:
            o = F.scaled_dot_product_attention(rotary(q), rotary(k), v)
            return self.o_proj(o.transpose(1, 2).reshape(n, l, -1)), None
        if cache is not None and l > 2:
            # a later SEGMENT of a long prompt: the cached window of the previous segment goes in front
            # (window and ALiBi bias are relative, so positions need no offset)
            kc, vc = torch.cat([cache[0], k], 2), torch.cat([cache[1], v], 2)
            qc = torch.cat([torch.zeros_like(cache[0]), q], 2)
            o = windowed_alibi_attention(qc, kc, vc, self.window, self.slopes)[:, :, -l:]
            new_cache = (kc[:, :, -(self.window + 1):], vc[:, :, -(self.window + 1):])
        elif cache is None:
            if torch.is_grad_enabled() and q.requires_grad:
                # SDPA with an explicit bias keeps the (window x 2 window) score blocks for its backward:
                # ~10 GB per layer at 8 x 16,640 positions.  Recompute them in the backward instead.
                from torch.utils.checkpoint import checkpoint
                o = checkpoint(windowed_alibi_attention, q, k, v, self.window, self.slopes, use_reentrant=False)
            else:
                o = windowed_alibi_attention(q, k, v, self.window, self.slopes)
            new_cache = (k[:, :, -(self.window + 1):], v[:, :, -(self.window + 1):]) if use_cache else None
        else:                                                    # a few new positions against the cached window
            kc, vc = torch.cat([cache[0], k], 2), torch.cat([cache[1], v], 2)
            t = kc.shape[2]
            if q.dtype == torch.bfloat16 and q.is_cuda and l <= 4 and self.d == 64 and not torch.is_grad_enabled():
                # the library's decode kernel for windowed ALiBi attention (flash_attn_with_kvcache in the reference)
                from . import fused_ops
                o = fused_ops.window_decode(q, kc, vc, self.window, self.slopes.float().contiguous(), 1.0 / math.sqrt(self.d))
                new_cache = (kc[:, :, -(self.window + 1):], vc[:, :, -(self.window + 1):])
                return self.o_proj(o.transpose(1, 2).reshape(n, l, -1)), new_cache
            qi = torch.arange(t - l, t, device=x.device).view(l, 1)
            kj = torch.arange(t, device=x.device).view(1, t)
            dist = (qi - kj).float()
            bias = (-self.slopes.view(self.h, 1, 1).float() * dist).masked_fill((dist < 0) | (dist > self.window), float("-inf"))
            o = F.scaled_dot_product_attention(q, kc, vc, attn_mask=bias.to(q.dtype).view(1, self.h, l, t))
            new_cache = (kc[:, :, -(self.window + 1):], vc[:, :, -(self.window + 1):])
        return self.o_proj(o.transpose(1, 2).reshape(n, l, -1)), new_cache


class DecoderLayer(nn.Module):
    def __init__(self, cfg: DRTConfig, bidirectional: bool = False):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.self_attn = SelfAttention(cfg, bidirectional)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.mlp = MLP(cfg)

    def forward(self, x, cache=None, use_cache=False):
        a, cache = self.self_attn(self.input_layernorm(x), cache, use_cache)
        x = x + a
        return x + self.mlp(self.post_attention_layernorm(x)), cache


class UpperDecoderLayer(nn.Module):
    """Self-attention, then GCA whose output joins the residual only as the MLP's input
    (``model/DRT.py:457-491``)."""

    def __init__(self, cfg: DRTConfig):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.self_attn = SelfAttention(cfg)
        self.gca = TritonGroupCrossAttention(cfg)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.mlp = MLP(cfg)
        self.chunk = cfg.enc_chunk_size + 1

    def forward(self, x, k_cache, v_cache, indices, weights, cache=None, use_cache=False, first_chunk_retrieves=False):
        a, cache = self.self_attn(self.input_layernorm(x), cache, use_cache)
        r = x + a
        n, l, dim = r.shape
        hs4 = r.view(n, l // self.chunk, self.chunk, dim) if l % self.chunk == 0 else r.view(n, 1, l, dim)
        if indices is None:                                       # nothing retrieved yet
            g = torch.zeros_like(r)
        else:
            g = self.gca.forward_indexed(hs4, k_cache, v_cache, indices, weights, first_chunk_retrieves)
        return r + self.mlp(self.post_attention_layernorm(r + g)), cache


class DecodeState:
    """Everything generation carries between steps."""

    def __init__(self, cfg: DRTConfig):
        self.self_attn: List[Optional[Tuple[torch.Tensor, torch.Tensor]]] = []
        self.chunks = ChunkKVManager(group_size=max(1, len(cfg.decoder_layers) - 1), zero_landmark=True)
        self.position = 0                                         # positions (tokens + landmarks) processed so far


class DRTMinimal(nn.Module):
    def __init__(self, cfg: DRTConfig):
        super().__init__()
        self.cfg = cfg
        self.chunk = cfg.enc_chunk_size + 1
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.lower_layers = nn.ModuleList(DecoderLayer(cfg) for _ in range(cfg.decoder_layers[0]))
        self.upper_layers = nn.ModuleList(nn.ModuleList(UpperDecoderLayer(cfg) for _ in range(nl)) for nl in cfg.decoder_layers[1:])
        self.lmk_norms = nn.ModuleList(RMSNorm(cfg.hidden_size, cfg.rms_norm_eps) for _ in cfg.decoder_layers[1:])
        self.enc_prenorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.encoder = nn.ModuleList(DecoderLayer(cfg, bidirectional=True) for _ in range(cfg.encoder_layers))
        self.encoder_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.chunk_k_proj = nn.Linear(cfg.hidden_size, cfg.hidden_size, bias=False)
        self.chunk_v_proj = nn.Linear(cfg.hidden_size, cfg.hidden_size, bias=False)
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        for m in self.modules():                                   # model/llama.py:842-851
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=cfg.initializer_range)

    # ------------------------------------------------------------------ pieces
    def insert_landmarks(self, tokens: torch.Tensor) -> torch.Tensor:
        """(N, T) with T a multiple of 63 -> (N, T / 63 * 64): the landmark id after every chunk."""
        n, t = tokens.shape
        if t % self.cfg.enc_chunk_size:
            raise ValueError(f"sequence length must be a multiple of {self.cfg.enc_chunk_size}")
        c = t // self.cfg.enc_chunk_size
        lmk = torch.full((n, c, 1), self.cfg.chunk_id, dtype=tokens.dtype, device=tokens.device)
        return torch.cat([tokens.view(n, c, -1), lmk], dim=2).view(n, c * self.chunk)

    def encode_chunks(self, hidden: torch.Tensor, chunks: ChunkKVManager) -> None:
        """hidden (N, C, 64, dim) lower-stack states of complete chunks: encode them and append K, V
        (projections of the encoder output, landmark rows zeroed) and the landmark embeddings (the encoder
        output's last row) to ``chunks`` -- one GEMM with the append as its epilogue when no gradient is
        needed (``ChunkKVManager.append_projected``)."""
        n, c, s, dim = hidden.shape
        x = self.enc_prenorm(hidden.reshape(n * c, s, dim))
        for layer in self.encoder:
            x, _ = layer(x)
        x = self.encoder_norm(x).view(n, c, s, dim)
        chunks.append_projected(x, self.chunk_k_proj.weight, self.chunk_v_proj.weight)

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return F.linear(self.norm(hidden), self.embed_tokens.weight)          # tied LM head

    # ------------------------------------------------------------------ full-sequence forward (training, prefill)
    def forward(self, tokens: torch.Tensor, labels: Optional[torch.Tensor] = None, state: Optional[DecodeState] = None):
        """tokens (N, T), T % 63 == 0.  Returns logits at token positions (N, T, vocab) -- or the loss when
        ``labels`` (N, T) are given (next-token targets are ``labels`` shifted left) -- and fills ``state``.
        A ``state`` that already holds earlier positions makes this call the NEXT SEGMENT of a long prompt
        (``model/DRT.py:1018-1050``): self-attention continues from the cached window, the chunk cache and
        landmarks grow, and the segment's first chunk uses the retrieval made at the end of the previous one."""
        cfg = self.cfg
        ids = self.insert_landmarks(tokens)
        n, l = ids.shape
        c = l // self.chunk
        x = self.embed_tokens(ids)
        use_cache = state is not None
        later = use_cache and state.position > 0
        old = state.self_attn if later else None
        caches = []
        for layer in self.lower_layers:
            x, kv = layer(x, old[len(caches)] if later else None, use_cache=use_cache)
            caches.append(kv)
        chunks = state.chunks if use_cache else ChunkKVManager(group_size=len(self.upper_layers), zero_landmark=True)
        self.encode_chunks(x.view(n, c, self.chunk, -1), chunks)
        for g, layers in enumerate(self.upper_layers):
            q_lmk = self.lmk_norms[g](x.view(n, c, self.chunk, -1)[:, :, -1])
            k = min(len(chunks), cfg.chunk_topk)
            idx, w, full = retrieve(q_lmk, chunks, k, training=self.training)
            if later:                                            # chunk 0 of this segment: the previous segment's last retrieval
                pidx, pw = chunks.current_retrieved_indices(g)
                pad = k - pidx.shape[-1]
                idx = torch.cat([F.pad(pidx, (0, pad), value=-1).unsqueeze(1), idx], dim=1)
                w = torch.cat([F.pad(pw, (0, pad)), w], dim=1)
            if use_cache:
                chunks.update_current_retrieved_chunk(full.indices, full.weights, g)
            have = later or c > 1
            for layer in layers:
                x, kv = layer(x, chunks.chunk_k, chunks.chunk_v, idx if have else None, w if have else None,
                              old[len(caches)] if later else None, use_cache=use_cache, first_chunk_retrieves=later)
                caches.append(kv)
        if use_cache:
            state.self_attn, state.position = caches, (state.position if later else 0) + l
        x = x.view(n, c, self.chunk, -1)[:, :, :-1].reshape(n, c * cfg.enc_chunk_size, -1)   # drop landmark positions
        if labels is None:
            return self.logits(x)
        target = torch.cat([labels[:, 1:], torch.full_like(labels[:, :1], -100)], dim=1).reshape(-1)
        # The (tokens x 50,265) logits of a 131,040-token batch are 26 GB in float32: the loss is summed over
        # pieces of 8,192 rows whose logits are recomputed in the backward instead of being kept.
        from torch.utils.checkpoint import checkpoint
        x = x.reshape(-1, x.shape[-1])
        if not torch.is_grad_enabled() and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 64 == 0:
            # evaluation: final norm + LM head + cross-entropy as one GEMM whose logits never leave tensor
            # memory (the norm's gain folded into the tied embedding matrix, 1 / rms applied per row)
            from . import fused_ops
            w = fused_ops.fold_gain(self.embed_tokens.weight.detach(), self.norm.weight.detach())
            losses = fused_ops.linear_cross_entropy(x, w, target, row_scale=fused_ops.row_rms(x, self.norm.eps))
            return losses.sum() / (target != -100).sum().clamp(min=1)

        def piece(xp, tp):
            return F.cross_entropy(self.logits(xp).float(), tp, ignore_index=-100, reduction="sum")

        total = x.new_zeros((), dtype=torch.float32)
        for r0 in range(0, x.shape[0], 8192):
            total = total + checkpoint(piece, x[r0:r0 + 8192], target[r0:r0 + 8192], use_reentrant=False)
        return total / (target != -100).sum().clamp(min=1)

    # ------------------------------------------------------------------ one decode step
    @torch.no_grad()
    def decode_step(self, token: torch.Tensor, state: DecodeState) -> torch.Tensor:
        """token (N,) -> logits (N, vocab) for the next token.  When the token completes a chunk the step
        also carries the landmark position: the chunk is encoded and appended, and the retrieval for the
        next chunk is made."""
        cfg = self.cfg
        boundary = (state.position + 1) % self.chunk == cfg.enc_chunk_size
        ids = token.view(-1, 1)
        if boundary:
            ids = torch.cat([ids, torch.full_like(ids, cfg.chunk_id)], dim=1)
        s = ids.shape[1]
        x = self.embed_tokens(ids)
        li = 0
        for layer in self.lower_layers:
            x, state.self_attn[li] = layer(x, state.self_attn[li])
            li += 1
        chunks = state.chunks
        chunks.cache_lower_hidden_states(x)
        if boundary:
            staged = chunks.lower_hidden_states                      # (N, 64, dim): the chunk is complete
            chunks.clear_lower_hidden_states()
            self.encode_chunks(staged.unsqueeze(1), chunks)
        for g, layers in enumerate(self.upper_layers):
            idx, w = chunks.current_retrieved_indices(g)             # fetched BEFORE this step's retrieval
            if boundary:
                q_lmk = self.lmk_norms[g](x[:, -1:])
                k = min(len(chunks), cfg.chunk_topk)
                res = lmk_score_topk(q_lmk, chunks.past_lmk_embeds, k)
                new_idx, new_w = res.indices[:, -1], res.weights[:, -1:]
            for layer in layers:
                x, state.self_attn[li] = layer(x, chunks.chunk_k, chunks.chunk_v,
                                               None if idx is None else idx.unsqueeze(1), w, state.self_attn[li])
                li += 1
            if boundary:
                chunks.update_current_retrieved_chunk(new_idx, new_w, g)
        state.position += s
        return self.logits(x[:, 0])

    @torch.no_grad()
    def prefill_segmented(self, prompt: torch.Tensor, segment_tokens: int, state: Optional[DecodeState] = None):
        """Prefill a long prompt segment by segment (``segment_tokens`` a multiple of 63), carrying the
        self-attention window and the growing chunk cache between segments, so that activation memory is
        bounded by the segment and not by the prompt (``model/DRT.py:1018-1050``,
        ``eval/slidewin_eval.py:115``; the reference parks the cache on the host meanwhile, here it stays
        in HBM).  Returns (logits of all token positions, state)."""
        if segment_tokens % self.cfg.enc_chunk_size:
            raise ValueError(f"segment length must be a multiple of {self.cfg.enc_chunk_size}")
        state = state or DecodeState(self.cfg)
        outs = [self.forward(prompt[:, t0:t0 + segment_tokens], state=state) for t0 in range(0, prompt.shape[1], segment_tokens)]
        return torch.cat(outs, dim=1), state

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, new_tokens: int) -> torch.Tensor:
        """Greedy decoding.  prompt (N, T), T % 63 == 0 (the reference left-pads the prompt to that,
        ``model/DRT.py:1149-1151``).  Returns (N, T + new_tokens)."""
        state = DecodeState(self.cfg)
        logits = self.forward(prompt, state=state)
        out = [prompt]
        tok = logits[:, -1].argmax(-1)
        for _ in range(new_tokens):
            out.append(tok.view(-1, 1))
            tok = self.decode_step(tok, state).argmax(-1)
        return torch.cat(out, dim=1)
