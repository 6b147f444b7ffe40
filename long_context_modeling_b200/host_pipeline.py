"""GCA forward + backward for callers whose tensors live in HOST memory.

A training step at the DRT-16K shape moves ~0.8 GB to the GPU (q, the two chunk caches, the
upstream gradient) and ~0.8 GB back (o, dq, dk, dv, dw) but computes for only ~2 ms, so a caller
that copies, computes and copies back in sequence spends >90 % of the step on PCIe in one
direction at a time.  `HostGcaPipeline` keeps `depth` steps in flight on three streams
(host->device, compute, device->host): the upload of step i+1, the kernels of step i and the
download of step i-1 overlap, and the link is used in both directions at once.

    pipe = HostGcaPipeline(device, sm_scale)
    for batch in batches:                      # pinned host tensors
        done = pipe.submit(batch)              # returns the finished outputs of an EARLIER step
        if done is not None: consume(done)     # (pinned host tensors), or None while filling
    for done in pipe.drain(): consume(done)

The math is `gca_indexed` and its autograd backward (same kernels, same results); only the
staging differs.  Mirrors nothing in the reference: there the tensors are already on the GPU
(`model/DRT.py:380`).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import gca as _gca


class HostGcaPipeline:
    def __init__(self, device: torch.device, sm_scale: float, depth: int = 2, softmax_off_by_one: bool = False):
        if depth < 2:
            raise ValueError("depth must be at least 2 (one step computing while another is copied)")
        self.device = torch.device(device)
        self.sm_scale = float(sm_scale)
        self.off_by_one = bool(softmax_off_by_one)
        self.depth = depth
        self.s_in = torch.cuda.Stream(self.device)
        self.s_comp = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        # `depth` sets of device inputs; one more set of pinned outputs, so that the set handed
        # back to the caller is not the one the step being submitted downloads into
        self._dev_in: List[Optional[Tuple[torch.Tensor, ...]]] = [None] * depth
        self._host_out: List[Optional[List[torch.Tensor]]] = [None] * (depth + 1)
        self._ev_in = [torch.cuda.Event() for _ in range(depth)]
        self._ev_comp = [torch.cuda.Event() for _ in range(depth)]
        self._ev_out = [torch.cuda.Event() for _ in range(depth + 1)]
        self._inflight: List[int] = []               # output slots of the steps not yet handed back
        self._count = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def _pop(self) -> List[torch.Tensor]:
        ob = self._inflight.pop(0)
        self._ev_out[ob].synchronize()
        # the step's kernels are complete: a bounded wait that expired in one of them means that
        # these outputs are not valid (raises GcaError)
        _gca.check_status(self.device)
        return self._host_out[ob]

    def submit(self, host: Sequence[torch.Tensor]) -> Optional[List[torch.Tensor]]:
        """host = (q, k_cache, v_cache, indices int32, weights float32, dout), pinned.

        Enqueues upload, forward + backward and download of this step.  Once `depth` steps are in
        flight it first waits for the oldest one and returns its outputs [o, dq, dk_cache,
        dv_cache, dw] (pinned host tensors, valid until the next call of `submit`); else None.
        """
        done = self._pop() if len(self._inflight) >= self.depth else None
        b = self._count % self.depth
        ob = self._count % (self.depth + 1)
        self._count += 1
        with torch.cuda.stream(self.s_in):
            if self._dev_in[b] is None:
                self._dev_in[b] = tuple(torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in host)
            self.s_in.wait_event(self._ev_comp[b])   # the kernels that last read these buffers are done
            for d, h in zip(self._dev_in[b], host):
                d.copy_(h, non_blocking=True)
            self._ev_in[b].record(self.s_in)
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in host)
        with torch.cuda.stream(self.s_comp):
            self.s_comp.wait_event(self._ev_in[b])
            dq_, dkc, dvc, didx, dw_, ddout = self._dev_in[b]
            qg = dq_.detach().requires_grad_()
            kg = dkc.detach().requires_grad_()
            vg = dvc.detach().requires_grad_()
            wg = dw_.detach().requires_grad_()
            o = _gca.gca_indexed(qg, kg, vg, didx, wg, self.sm_scale, softmax_off_by_one=self.off_by_one)
            o.backward(ddout)
            outs = [o.detach(), qg.grad, kg.grad, vg.grad, wg.grad]
            self._ev_comp[b].record(self.s_comp)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self._ev_comp[b])
            if self._host_out[ob] is None:
                self._host_out[ob] = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in outs]
            for h, d in zip(self._host_out[ob], outs):
                h.copy_(d, non_blocking=True)
                d.record_stream(self.s_out)
            self._ev_out[ob].record(self.s_out)
        self.d2h_bytes = sum(t.numel() * t.element_size() for t in outs)
        self._inflight.append(ob)
        return done

    def drain(self) -> List[List[torch.Tensor]]:
        """Waits for every step still in flight; returns their outputs, oldest first (each valid
        until the next call of `submit`)."""
        res = []
        while self._inflight:
            res.append(self._pop())
        return res
