"""GPU-resident chunk K/V + landmark cache: mirror of ``ChunkKVManager``
(``model/DRT.py:75-233``).

The reference grows its cache with ``torch.cat`` on every append (quadratic copying over a
long generation) and can park K/V on the host.  Here the cache is a preallocated device
buffer that is filled in place by one CUDA kernel per append and doubled when full -- or, with
``max_chunks``, a virtual-address reservation behind which memory is mapped as the cache fills, so
that nothing is ever re-copied and addresses never change (``virtual_memory.py``); the
kernels read it by chunk index, so ``retrieve_chunks`` (the materialised gather) is needed
only by callers that want the reference's gathered tensors.  The public methods keep the
reference's names and argument meaning.

Training.  The reference's manager keeps the autograd tensors it is given
(``model/DRT.py:87-133,784``), so gradients flow from GCA and from the retrieval weights back
into ``chunk_k_proj`` / ``chunk_v_proj``, the chunk encoder and the cached landmarks.  The
in-place buffer would cut that graph, so an ``append`` whose inputs require grad (with grad
mode on) switches the manager to a FUNCTIONAL mode: the appended tensors themselves are kept
(one append per forward pass, as in the reference's training step, is stored without any copy;
further appends are concatenated with ``torch.cat`` like the reference's), ``chunk_k``,
``chunk_v`` and ``past_lmk_embeds`` return them, and ``gca_indexed`` / ``retrieve`` on those
tensors back-propagate into the caller's graph.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Tuple

import torch

from . import _lib


class ChunkKVManager:
    def __init__(self, offloading: bool = False, group_size: int = 1, capacity: int = 0,
                 zero_landmark: bool = False, max_chunks: int = 0):
        # `offloading` is accepted for signature compatibility; the cache always stays in
        # device memory (180 GB of HBM hold > 50 sequences of 1M tokens at DRT-small scale).
        self._offloading = offloading
        self.group_size = group_size
        self._capacity_hint = capacity
        self._zero_landmark = zero_landmark
        # max_chunks > 0: K and V live in a virtual-address reservation for that many chunks per sequence
        # and physical memory is mapped behind it as the cache fills (no copy on growth, ever)
        self._max_chunks = int(max_chunks)
        self._vk = self._vv = None
        self._mapped = 0                             # chunks per sequence that are backed by memory (virtual mode)
        self._k: Optional[torch.Tensor] = None       # (N, capacity, L, HD)
        self._v: Optional[torch.Tensor] = None
        self._lmk: Optional[torch.Tensor] = None     # (N, capacity, Dm)
        self._len = 0
        self._grad_mode = False                      # functional storage: the tensors below carry autograd history
        self._gk: Optional[torch.Tensor] = None
        self._gv: Optional[torch.Tensor] = None
        self._glmk: Optional[torch.Tensor] = None
        self._cur_idx: List[Optional[torch.Tensor]] = [None] * group_size
        self._cur_w: List[Optional[torch.Tensor]] = [None] * group_size
        self._current_hidden_states = None

    # ------------------------------------------------------------------ storage
    def __len__(self) -> int:
        return self._len

    @property
    def chunk_k(self) -> Optional[torch.Tensor]:
        if self._grad_mode:
            return self._gk
        return None if self._k is None else self._k[:, :self._len]

    @property
    def chunk_v(self) -> Optional[torch.Tensor]:
        if self._grad_mode:
            return self._gv
        return None if self._v is None else self._v[:, :self._len]

    @property
    def lmk_embs(self) -> Optional[torch.Tensor]:
        if self._grad_mode:
            return self._glmk
        return None if self._lmk is None else self._lmk[:, :self._len]

    def backed_views(self):
        """(chunk_k, chunk_v) over EVERY chunk slot that has memory behind it, filled or not: a view whose
        address and shape stay the same while chunks are appended (until the buffer is re-allocated or the
        next pages are mapped), for callers that bake tensor arguments into a CUDA graph.  Only chunks
        below ``len(self)`` hold data; retrieved indices never point past them."""
        if self._grad_mode or self._k is None:
            return self.chunk_k, self.chunk_v
        cap = self._capacity()
        return self._k[:, :cap], self._v[:, :cap]

    @property
    def tracks_gradients(self) -> bool:
        """True once an append with grad-requiring inputs switched the manager to functional storage."""
        return self._grad_mode

    def _append_functional(self, chunk_k: torch.Tensor, chunk_v: torch.Tensor, lmk_embs: torch.Tensor) -> None:
        if self._zero_landmark:                   # the landmark row of every chunk is cleared (model/DRT.py:771-781)
            keep = torch.ones(chunk_k.shape[-2], 1, dtype=chunk_k.dtype, device=chunk_k.device)
            keep[-1] = 0
            chunk_k, chunk_v = chunk_k * keep, chunk_v * keep
        if not self._grad_mode:
            self._grad_mode = True
            if self._len:                         # what the buffer holds so far joins as constants
                self._gk, self._gv = self._k[:, :self._len].clone(), self._v[:, :self._len].clone()
                self._glmk = self._lmk[:, :self._len].clone()
            self._k = self._v = self._lmk = None
            for vb in (self._vk, self._vv):       # a virtual reservation is given back: functional storage from here on
                if vb is not None:
                    vb.close()
            self._vk = self._vv = None
            self._max_chunks = self._mapped = 0
        if self._gk is None:
            self._gk, self._gv, self._glmk = chunk_k, chunk_v, lmk_embs
        else:
            self._gk = torch.cat([self._gk, chunk_k.to(self._gk.dtype)], dim=1)
            self._gv = torch.cat([self._gv, chunk_v.to(self._gv.dtype)], dim=1)
            self._glmk = torch.cat([self._glmk, lmk_embs.to(self._glmk.dtype)], dim=1)
        self._len += chunk_k.shape[1]

    @property
    def past_lmk_embeds(self) -> Optional[torch.Tensor]:
        return self.lmk_embs

    def _capacity(self) -> int:
        """Chunks per sequence the K / V buffers can hold right now."""
        if self._vk is not None:
            return self._mapped
        return 0 if self._k is None else self._k.shape[1]

    def _reserve_virtual(self, need: int, like_k: torch.Tensor, like_lmk: torch.Tensor) -> None:
        from .virtual_memory import VirtualBuffer
        n, _, l, hd = like_k.shape
        if need > self._max_chunks:
            raise ValueError(f"the cache was reserved for {self._max_chunks} chunks per sequence, {need} needed")
        chunk_bytes = l * hd * like_k.element_size()
        if self._vk is None:
            self._vk = VirtualBuffer(like_k.device, n, self._max_chunks * chunk_bytes)
            self._vv = VirtualBuffer(like_k.device, n, self._max_chunks * chunk_bytes)
            self._k, self._v = self._vk.view(like_k.dtype, (l, hd)), self._vv.view(like_k.dtype, (l, hd))
        if need > self._mapped:
            want = max(need, min(self._max_chunks, self._mapped + max(16, self._capacity_hint)))     # grow in steps, not per append
            self._vv.ensure(want * chunk_bytes)
            self._mapped = self._vk.ensure(want * chunk_bytes) // chunk_bytes
        cap = 0 if self._lmk is None else self._lmk.shape[1]
        if need > cap:                                # landmarks are 1.5 KB per chunk: a plain doubling buffer
            lmk = torch.empty((n, min(self._max_chunks, max(need, 2 * cap, 64)), like_lmk.shape[-1]), dtype=like_lmk.dtype,
                              device=like_lmk.device)
            if self._len:
                lmk[:, :self._len].copy_(self._lmk[:, :self._len])
            self._lmk = lmk

    def close(self) -> None:
        """Give the cache's memory back (virtual mode: unmap and release the reservation)."""
        self._k = self._v = self._lmk = None
        for vb in (self._vk, self._vv):
            if vb is not None:
                vb.close()
        self._vk = self._vv = None
        self._len = self._mapped = 0

    def _reserve(self, need: int, like_k: torch.Tensor, like_lmk: torch.Tensor) -> None:
        if self._max_chunks:
            return self._reserve_virtual(need, like_k, like_lmk)
        cap = 0 if self._k is None else self._k.shape[1]
        if need <= cap:
            return
        new_cap = max(need, 2 * cap, self._capacity_hint, 16)
        n, _, l, hd = like_k.shape
        k = torch.empty((n, new_cap, l, hd), dtype=like_k.dtype, device=like_k.device)
        v = torch.empty_like(k)
        lmk = torch.empty((n, new_cap, like_lmk.shape[-1]), dtype=like_lmk.dtype, device=like_lmk.device)
        if self._len:
            k[:, :self._len].copy_(self._k[:, :self._len])
            v[:, :self._len].copy_(self._v[:, :self._len])
            lmk[:, :self._len].copy_(self._lmk[:, :self._len])
        self._k, self._v, self._lmk = k, v, lmk

    def append(self, chunk_k: torch.Tensor, chunk_v: torch.Tensor, lmk_embs: torch.Tensor) -> None:
        """chunk_k, chunk_v (N, D, S, dim); lmk_embs (N, D, dim)  (``model/DRT.py:87-133``)."""
        if not chunk_k.is_cuda:
            raise RuntimeError("ChunkKVManager holds device memory only (there is no CPU path)")
        if chunk_k.shape != chunk_v.shape or chunk_k.dim() != 4 or lmk_embs.dim() != 3:
            raise ValueError("expected chunk_k/chunk_v (N, D, S, dim) and lmk_embs (N, D, dim)")
        if self._k is not None and (chunk_k.shape[-2] != self._k.shape[-2] or chunk_k.shape[0] != self._k.shape[0]):
            raise ValueError("chunk shape does not match the cache")
        if self._grad_mode or (torch.is_grad_enabled() and
                               (chunk_k.requires_grad or chunk_v.requires_grad or lmk_embs.requires_grad)):
            self._append_functional(chunk_k, chunk_v, lmk_embs)
            return
        if self._k is not None:
            chunk_k, chunk_v = chunk_k.to(self._k.dtype), chunk_v.to(self._k.dtype)
            lmk_embs = lmk_embs.to(self._lmk.dtype)
        chunk_k, chunk_v, lmk_embs = chunk_k.contiguous(), chunk_v.contiguous(), lmk_embs.contiguous()
        n, count, l, hd = chunk_k.shape
        self._reserve(self._len + count, chunk_k, lmk_embs)
        if chunk_k.dtype != lmk_embs.dtype:
            # landmarks kept in another precision than K/V: two launches of the same kernel path
            self._lmk[:, self._len:self._len + count].copy_(lmk_embs)
            lmk_src = None
        else:
            lmk_src = lmk_embs
        a = _lib.CacheAppendArgs()
        a.new_k, a.new_v = chunk_k.data_ptr(), chunk_v.data_ptr()
        a.k_cache, a.v_cache = self._k.data_ptr(), self._v.data_ptr()
        a.new_lmk = lmk_src.data_ptr() if lmk_src is not None else None
        a.lmk_cache = self._lmk.data_ptr() if lmk_src is not None else None
        a.new_batch_stride, a.cache_batch_stride = chunk_k.stride(0), self._k.stride(0)
        a.new_lmk_batch_stride, a.lmk_cache_batch_stride = lmk_embs.stride(0), self._lmk.stride(0)
        a.N, a.count, a.pos, a.L, a.HD, a.Dm = n, count, self._len, l, hd, lmk_embs.shape[-1]
        a.dtype = _lib.BF16 if chunk_k.dtype == torch.bfloat16 else _lib.F32
        if chunk_k.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"unsupported cache dtype {chunk_k.dtype}")
        a.zero_landmark = 1 if self._zero_landmark else 0
        a.capacity, a.lmk_capacity = self._capacity(), self._lmk.shape[1]
        with torch.cuda.device(chunk_k.device):
            _lib.call("gca_cache_append", C.byref(a), torch.cuda.current_stream().cuda_stream)
        self._len += count

    def append_projected(self, enc_out: torch.Tensor, k_weight: torch.Tensor, v_weight: torch.Tensor) -> None:
        """The reference's ``chunk_k_proj`` / ``chunk_v_proj`` + landmark extraction + ``append``
        (``model/DRT.py:766-784``) as ONE tensor-core GEMM whose epilogue writes K and V straight into
        the cache (landmark rows cleared when the manager was built with ``zero_landmark``) and the
        landmark rows of ``enc_out`` into the landmark cache.  enc_out (N, D, 64, dim) bf16; the weights
        are the two ``nn.Linear.weight`` tensors (dim, dim), no bias.  Inference path: when the inputs
        require grad the projections are done with torch and ``append`` keeps the graph."""
        if (torch.is_grad_enabled() and (enc_out.requires_grad or k_weight.requires_grad or v_weight.requires_grad)) or \
                self._grad_mode or enc_out.dtype != torch.bfloat16 or enc_out.shape[-1] % 256 != 0 or enc_out.shape[-2] != 64:
            x = enc_out
            self.append(torch.nn.functional.linear(x, k_weight), torch.nn.functional.linear(x, v_weight), x[:, :, -1])
            return
        if not enc_out.is_cuda:
            raise RuntimeError("ChunkKVManager holds device memory only (there is no CPU path)")
        x = enc_out.contiguous()
        n, count, l, dim = x.shape
        self._reserve(self._len + count, x, x[:, :, -1])
        if self._k.dtype != torch.bfloat16 or self._lmk.dtype != torch.bfloat16:
            raise ValueError("append_projected writes a bf16 cache")
        a = _lib.KvProjectArgs()
        a.x, a.wk, a.wv = x.data_ptr(), k_weight.contiguous().data_ptr(), v_weight.contiguous().data_ptr()
        a.k_cache, a.v_cache, a.lmk_cache = self._k.data_ptr(), self._v.data_ptr(), self._lmk.data_ptr()
        from .gca import _status
        a.status = _status(x.device).data_ptr()
        a.cache_batch_stride, a.lmk_cache_batch_stride = self._k.stride(0), self._lmk.stride(0)
        a.N, a.count, a.pos, a.D = n, count, self._len, dim
        a.capacity, a.lmk_capacity = self._capacity(), self._lmk.shape[1]
        a.zero_landmark = 1 if self._zero_landmark else 0
        with torch.cuda.device(x.device):
            _lib.call("gca_kv_project_append", C.byref(a), torch.cuda.current_stream().cuda_stream)
        self._len += count

    # ------------------------------------------------------------------ retrieval state
    def retrieve_chunks(self, indices: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """indices (N, M) -> gathered k, v (N, M, S, dim)  (``model/DRT.py:193-199``).
        Compatibility path: the GCA kernels read the cache by index and do not need this."""
        n = indices.shape[0]
        batch = torch.arange(n, device=indices.device).unsqueeze(1)
        idx = indices.clamp(min=0).long()
        return self.chunk_k[batch, idx], self.chunk_v[batch, idx]

    def update_current_retrieved_chunk(self, indices: torch.Tensor, weights: torch.Tensor, group_idx: int) -> None:
        """Remember the chunks retrieved for the tokens to come (``model/DRT.py:158-191``):
        indices (N, K) or (N, Cq, K) (last row is used); weights (N, Cq, K)."""
        if indices.dim() == 3:
            indices = indices[:, -1, :]
        self._cur_idx[group_idx] = indices.to(torch.int32).contiguous()
        self._cur_w[group_idx] = weights[:, -1:, :].to(torch.float32).contiguous()

    def current_retrieved_indices(self, group_idx: int = 0):
        """(indices (N, K) int32 with -1 padding, weights (N, 1, K)) for ``gca_indexed``."""
        return self._cur_idx[group_idx], self._cur_w[group_idx]

    def current_retrieved_chunk(self, group_idx: int = 0):
        """Gathered (chunk_k (N, K, S, dim), chunk_v, weights (N, 1, K)) like the reference
        (``model/DRT.py:139-140``); materialised on demand."""
        idx, w = self._cur_idx[group_idx], self._cur_w[group_idx]
        if idx is None:
            return None, None, None
        k, v = self.retrieve_chunks(idx)
        return k, v, w

    # ------------------------------------------------------------------ lower hidden-state staging
    @property
    def lower_hidden_states(self):
        return self._current_hidden_states

    def clear_lower_hidden_states(self) -> None:
        self._current_hidden_states = None

    def cache_lower_hidden_states(self, hidden_states: torch.Tensor) -> None:
        if self._current_hidden_states is None:
            self._current_hidden_states = hidden_states
        else:
            self._current_hidden_states = torch.cat([self._current_hidden_states, hidden_states], dim=1)
