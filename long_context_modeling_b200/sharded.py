"""Chunk-range-sharded landmark retrieval and GCA decode for very long contexts.

The reference never shards retrieval (it parks the chunk cache on the host instead,
``model/DRT.py:87-128`` and ``eval/slidewin_eval.py:115``).  Here rank ``r`` of ``g`` owns
the contiguous chunk range ``shard_range(E, g, r)`` of the landmark and K/V cache.  A
retrieval step is

1. local: fused score + top-k over the local landmarks, reporting GLOBAL chunk ids
   (``lmk_score_topk(..., e_base=lo)``),
2. exchange: ONE all-gather of the ``K`` packed 64-bit candidates per row (NCCL over
   NVLink; 64 B per row per rank for K = 8),
3. merge: every rank selects the same global top-k from the ``g*K`` candidates (integer
   order on the packed keys, so the result is identical everywhere).

With a ``PeerExchange`` steps 2 and 3 are ONE kernel launch per rank: each rank stores its
candidates straight into every rank's mailbox through CUDA IPC peer mappings, raises a flag,
waits (bounded) for the others and merges; ``ShardedRetriever`` replays scan + exchange from a
CUDA graph.  The NCCL path stays as the checked reference of the exchange.

GCA over the winners is owner-computes: each rank attends over the winners it holds, with
the globally normalised weights, and the (tiny) outputs are summed with an all-reduce.

Failures are detected on the host: every payload carries a header (rank, rows, K, range)
that is checked after the exchange; a rank that never joins ends the collective with the
process group's timeout.  Both surface as ``ShardExchangeError``.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib
from .gca import _status
from .retrieval import Retrieval, lmk_score_topk, merge_topk

HEADER = 6          # rank, rows, K, lo, hi, magic
MAGIC = 0x6C6D6B31  # "lmk1"


class ShardExchangeError(RuntimeError):
    pass


def shard_range(e_total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced chunk range [lo, hi) owned by ``rank``."""
    base, rem = divmod(e_total, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def _decode_scores(keys: torch.Tensor) -> torch.Tensor:
    """Float32 scores of packed keys held in a CPU int64 tensor (host-side check only)."""
    import numpy as np
    k = keys.contiguous().numpy().view(np.uint64)
    o = (k >> np.uint64(32)).astype(np.uint32)
    neg = (o >> np.uint32(31)) == 0
    bits = np.where(neg, ~o, o & np.uint32(0x7FFFFFFF)).astype(np.uint32)
    return torch.from_numpy(bits.view(np.float32).copy())


def validate_payloads(payloads, world: int, rows: int, topk: int, e_total: int) -> None:
    """Check what the exchange delivered; raises ShardExchangeError naming the first fault."""
    if len(payloads) != world:
        raise ShardExchangeError(f"expected {world} payloads, got {len(payloads)}")
    for r, p in enumerate(payloads):
        p = p.cpu()
        if p.numel() != HEADER + rows * topk:
            raise ShardExchangeError(f"rank {r}: payload has {p.numel()} words, expected {HEADER + rows * topk}")
        h = p[:HEADER].tolist()
        if h[5] != MAGIC:
            raise ShardExchangeError(f"rank {r}: payload missing or corrupt (bad magic)")
        if h[0] != r:
            raise ShardExchangeError(f"rank {r}: payload claims to come from rank {h[0]}")
        if h[1] != rows or h[2] != topk:
            raise ShardExchangeError(f"rank {r}: rows/k mismatch ({h[1]}, {h[2]}) vs ({rows}, {topk})")
        lo, hi = shard_range(e_total, world, r)
        if (h[3], h[4]) != (lo, hi):
            raise ShardExchangeError(f"rank {r}: owns [{h[3]}, {h[4]}) but the plan says [{lo}, {hi})")
        keys = p[HEADER:]
        live = keys != 0
        idx = 0xFFFFFFFF - (keys & 0xFFFFFFFF)
        if bool(((idx < lo) | (idx >= hi))[live].any()):
            raise ShardExchangeError(f"rank {r}: candidate outside its chunk range [{lo}, {hi})")
        scores = _decode_scores(keys[live])
        if bool(torch.isnan(scores).any()):
            raise ShardExchangeError(f"rank {r}: NaN score among the candidates")


def sharded_lmk_topk(lmk_q: torch.Tensor, lmk_k_local: torch.Tensor, topk: int, *, e_total: int,
                     group=None, head_dim: int = 0, q_pos0: Optional[int] = None, validate: bool = True,
                     score_fn: Callable = lmk_score_topk, merge_fn: Callable = merge_topk,
                     _tamper: Optional[Callable] = None, exchange: Optional["PeerExchange"] = None) -> Retrieval:
    """Global top-k over a landmark cache sharded by chunk range.

    lmk_q (N, Cq, D) replicated on every rank; lmk_k_local (N, hi-lo, D) this rank's range.
    ``q_pos0`` defaults to ``e_total - Cq`` (the reference's causal mask over the whole
    cache).  ``score_fn`` / ``merge_fn`` default to the CUDA kernels; tests running CPU
    ranks inject checkers.  ``_tamper`` lets a test corrupt this rank's payload.
    ``exchange`` (a ``PeerExchange``) replaces the NCCL all-gather and the merge launch by the
    fused peer-store exchange kernel; without it the step is local scan -> all-gather -> merge.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    lo, hi = shard_range(e_total, world, rank)
    if lmk_k_local.shape[1] != hi - lo:
        raise ValueError(f"rank {rank} must hold chunks [{lo}, {hi}), got {lmk_k_local.shape[1]} landmarks")
    cq = lmk_q.shape[1]
    q_pos0 = (e_total - cq) if q_pos0 is None else q_pos0
    local = score_fn(lmk_q, lmk_k_local, topk, q_pos0=q_pos0, e_base=lo, head_dim=head_dim)
    rows_shape = tuple(local.keys.shape[:-1])
    rows = 1
    for s in rows_shape:
        rows *= s
    if exchange is not None:
        return exchange.exchange(local.keys, topk)
    if not validate and _tamper is None:
        # lean path (no payload header, no host-side checks): one all-gather of the packed keys
        # into a (world, rows, K) buffer; for a single row that buffer already is the merge input
        gathered = torch.empty((world, rows, topk), dtype=torch.int64, device=local.keys.device)
        try:
            dist.all_gather_into_tensor(gathered, local.keys.reshape(rows, topk).contiguous(), group=group)
        except RuntimeError as exc:
            raise ShardExchangeError(f"candidate exchange failed: {exc}") from exc
        keys = gathered.view(1, world * topk) if rows == 1 else gathered.permute(1, 0, 2).reshape(rows, world * topk)
        return merge_fn(keys.reshape(rows_shape + (world * topk,)), topk)
    header = torch.tensor([rank, rows, topk, lo, hi, MAGIC], dtype=torch.int64, device=local.keys.device)
    payload = torch.cat([header, local.keys.reshape(-1)])
    if _tamper is not None:
        payload = _tamper(payload)
    gathered = [torch.empty(HEADER + rows * topk, dtype=torch.int64, device=payload.device) for _ in range(world)]
    try:
        if payload.numel() != HEADER + rows * topk:
            # a malformed local payload would make the collective itself undefined: send a
            # well-sized poison record instead so every rank fails the same check
            payload = torch.zeros(HEADER + rows * topk, dtype=torch.int64, device=payload.device)
        dist.all_gather(gathered, payload.contiguous(), group=group)
    except RuntimeError as exc:          # a rank never joined / left: the group timed out
        raise ShardExchangeError(f"candidate exchange failed: {exc}") from exc
    if validate:
        validate_payloads(gathered, world, rows, topk, e_total)
    keys = torch.stack([g[HEADER:].view(rows, topk) for g in gathered], dim=1).reshape(rows_shape + (world * topk,))
    return merge_fn(keys, topk)


class PeerExchange:
    """Mailboxes for the fused candidate exchange among the GPUs of one node (``lmk_topk_exchange``
    in the C ABI): every rank allocates a mailbox, the ranks swap CUDA IPC handles through the
    process group (host side, once), and each maps the others' mailboxes.  One ``exchange`` call is
    ONE kernel launch per rank: it stores this rank's candidates into every mailbox, raises a flag,
    waits (bounded by ``wait_ms``) for the other ranks' flags and merges.  No collective library is
    involved in a step, so the step can be captured in a CUDA graph (``ShardedRetriever``).

    A step in which some rank never publishes ends on the others with ``GCA_STATUS_TIMEOUT`` in the
    status word (``check_status`` raises ``GcaError``); afterwards call ``reset()`` on every rank.
    """

    def __init__(self, device: torch.device, max_rows: int, group=None, wait_ms: int = 1000):
        self.group, self.device, self.r_max, self.wait_ms = group, torch.device(device), int(max_rows), int(wait_ms)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        lib = _lib.lib()
        handle = (C.c_uint8 * 64)()
        own = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.call("lmk_exchange_mailbox_create", self.r_max, self.world, C.byref(own), handle)
        self._own = own.value
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)          # host-side swap of the 64-byte handles
        self._peers = []
        ptrs = []
        with torch.cuda.device(self.device):
            for r, h in enumerate(handles):
                if r == self.rank:
                    ptrs.append(self._own)
                    continue
                buf = (C.c_uint8 * 64).from_buffer_copy(h)
                peer = C.c_void_p()
                _lib.call("lmk_exchange_mailbox_open", buf, C.byref(peer))
                self._peers.append(peer.value)
                ptrs.append(peer.value)
        self._table = torch.tensor(ptrs, dtype=torch.int64, device=self.device)     # the device array of mailbox pointers
        dist.barrier(group=group)                # every mailbox is mapped everywhere before the first step

    def exchange(self, local_keys: torch.Tensor, topk: int) -> Retrieval:
        """local_keys (..., K) packed candidates of this rank -> the global top-k per row."""
        keys = local_keys.contiguous()
        rows_shape = tuple(keys.shape[:-1])
        rows = 1
        for s_ in rows_shape:
            rows *= s_
        dev = keys.device
        out_keys = torch.empty(rows_shape + (topk,), dtype=torch.int64, device=dev)
        indices = torch.empty(rows_shape + (topk,), dtype=torch.int32, device=dev)
        scores = torch.empty(rows_shape + (topk,), dtype=torch.float32, device=dev)
        weights = torch.empty(rows_shape + (topk,), dtype=torch.float32, device=dev)
        n_valid = torch.empty(rows_shape, dtype=torch.int32, device=dev)
        a = _lib.LmkExchangeArgs()
        a.local_keys, a.mailboxes = keys.data_ptr(), self._table.data_ptr()
        a.out_keys, a.out_indices, a.out_scores = out_keys.data_ptr(), indices.data_ptr(), scores.data_ptr()
        a.out_weights, a.out_nvalid = weights.data_ptr(), n_valid.data_ptr()
        a.status = _status(dev).data_ptr()
        a.R, a.K, a.world, a.rank, a.R_max, a.wait_ms = rows, int(topk), self.world, self.rank, self.r_max, self.wait_ms
        with torch.cuda.device(dev):
            _lib.call("lmk_topk_exchange", C.byref(a), torch.cuda.current_stream().cuda_stream)
        return Retrieval(out_keys, indices, scores, weights, n_valid)

    def reset(self) -> None:
        """After a failed step: all ranks meet on the host, then every mailbox (and its step counters)
        is cleared, then they meet again before anybody publishes."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            _lib.call("lmk_exchange_mailbox_reset", self._own, self.r_max, self.world,
                                                             torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def close(self) -> None:
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)           # nobody still stores into a mailbox that is about to go
        lib = _lib.lib()
        with torch.cuda.device(self.device):
            for p_ in self._peers:
                lib.lmk_exchange_mailbox_close(p_)
            dist.barrier(group=self.group)
            lib.lmk_exchange_mailbox_destroy(self._own)
        self._own, self._peers = None, []


class ShardedRetriever:
    """The sharded retrieval step (local scan -> fused peer-store exchange + merge) for a FIXED
    problem shape, captured once in a CUDA graph and replayed per query.

    At 16M tokens over 8 GPUs the local scan is ~10 us of HBM time, while three kernel launches
    issued from Python cost ~60 us of host time per step: eager, the sharded step is slower than
    the one-GPU scan it is meant to beat.  Replayed from a graph the step costs its device time
    only.  The graph holds this repository's kernels only (no collective library call), every rank
    must replay the same number of times, the query landmark is copied into a static buffer before
    each replay and the result tensors are reused: read them before the next call.
    """

    def __init__(self, lmk_q_like: torch.Tensor, lmk_k_local: torch.Tensor, topk: int, *, e_total: int,
                 exchange: PeerExchange, head_dim: int = 0, q_pos0: Optional[int] = None):
        self.exchange, self.topk, self.e_total, self.head_dim, self.q_pos0 = exchange, topk, e_total, head_dim, q_pos0
        self.lk = lmk_k_local
        self.lq = torch.empty_like(lmk_q_like)
        self.lq.copy_(lmk_q_like)
        for _ in range(2):                      # lazy initialisation happens outside the capture
            self._step()
        torch.cuda.synchronize(self.lq.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.result = self._step()

    def _step(self) -> Retrieval:
        return sharded_lmk_topk(self.lq, self.lk, self.topk, e_total=self.e_total, group=self.exchange.group,
                                head_dim=self.head_dim, q_pos0=self.q_pos0, exchange=self.exchange)

    def __call__(self, lmk_q: torch.Tensor) -> Retrieval:
        self.lq.copy_(lmk_q, non_blocking=True)
        self.graph.replay()
        return self.result


def sharded_gca_decode(q: torch.Tensor, k_cache_local: torch.Tensor, v_cache_local: torch.Tensor,
                       indices: torch.Tensor, weights: torch.Tensor, sm_scale: float, *, e_total: int,
                       group=None, gca_fn: Optional[Callable] = None) -> torch.Tensor:
    """Owner-computes GCA over a K/V cache sharded by chunk range.

    q (N, 1, Hq, Sq, D) replicated; caches hold this rank's chunks [lo, hi); indices are
    GLOBAL chunk ids (N, 1, K) with -1 padding and weights the globally normalised
    retrieval weights.  Every rank attends over the winners it owns (the others become
    padding slots), then the partial outputs are summed across ranks."""
    if gca_fn is None:
        from .gca import gca_indexed_nograd as gca_fn
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    lo, hi = shard_range(e_total, world, rank)
    mine = (indices >= lo) & (indices < hi)
    local_idx = torch.where(mine, indices - lo, torch.full_like(indices, -1))
    part = gca_fn(q, k_cache_local, v_cache_local, local_idx, weights, sm_scale).float()
    dist.all_reduce(part, group=group)
    return part.to(q.dtype)
