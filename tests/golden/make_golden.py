"""Generate the golden fixtures in this directory by running the REFERENCE's own source.

The reference project cannot be imported as a package without a GPU (its Triton file
queries the driver at import, its model file imports absent third-party extensions), so
this script lifts the pure-PyTorch pieces out of the reference checkout *by source text*
and executes them on CPU tensors:

* ``ltriton/gca.py`` -- the einsum ground truth inside ``test_group_qa`` (the lines from
  ``k_ = torch.repeat_interleave`` to ``ref_out = torch.einsum(...)``), plus autograd.
* ``model/DRT.py``   -- class ``ChunkKVManager``, ``DRT._enc_dec_score_mask``,
  ``DRT._perform_batch_retrieval``, ``TritonGroupCrossAttention.preprocess_chunk_kv_cache``
  (lifted with ``ast``), and the decode-time retrieval statements inside ``DRT.forward``.
* ``model/DRT.py``   -- the whole classes ``TritonGroupCrossAttention`` and
  ``GroupCrossAttention`` (constructor, ``preprocess_chunk_kv_cache``, ``forward``), executed
  with stand-ins for the three third-party callables they use: the fused ``RMSNorm`` (plain
  formula), ``gca_attn`` / ``gca_kv_cache`` (the reference's einsum ground truth lifted above)
  and ``flash_attn_func`` (plain softmax attention).  What the fixture pins is the glue: norm,
  projection, head split, dropping the first chunk, the K-fold query expansion of the flash
  variant, the weighted merge, the output projection and the zero rows of the first chunk.

Usage (only where the reference checkout exists):
    python tests/golden/make_golden.py /path/to/reference
Outputs ``*.npz`` next to this file.  Nothing is copied from the reference into the
repository: only numeric outputs are stored.
"""
from __future__ import annotations

import ast
import math
import os
import sys
import textwrap

import numpy as np
import torch
import torch.nn.functional as F
from einops import rearrange, repeat

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def _slice_between(src: str, first: str, last: str, occurrence: int = 0) -> str:
    lines = src.splitlines()
    starts = [i for i, ln in enumerate(lines) if first in ln]
    i0 = starts[occurrence]
    i1 = next(i for i in range(i0, len(lines)) if last in lines[i])
    return textwrap.dedent("\n".join(lines[i0:i1 + 1]))


def reference_einsum_block(ref_root: str, group: int) -> str:
    src = open(os.path.join(ref_root, "ltriton", "gca.py")).read()
    block = _slice_between(src, "k_ = torch.repeat_interleave(k, dim=1, repeats=4)",
                           "ref_out = torch.einsum('Z H K M h, Z K->Z H M h', o_k, weights)")
    # the reference hard-codes its test's GQA group (4); the group is the only edit
    return block.replace("repeats=4", f"repeats={group}")


def run_reference_gca(block: str, q, k, v, w, sm_scale, dout, dtype):
    q = q.clone().requires_grad_()
    k = k.clone().requires_grad_()
    v = v.clone().requires_grad_()
    w = w.clone().requires_grad_()
    ns = dict(torch=torch, q=q, k=k, v=v, weights=w, sm_scale=sm_scale, dtype=dtype)
    exec(block, ns)
    ref_out = ns["ref_out"]
    ref_out.backward(dout)
    return ref_out.detach(), q.grad, k.grad, v.grad, w.grad


def lift_reference_retrieval(ref_root: str):
    """Returns (ChunkKVManager, DummyDRT class, decode_block source)."""
    src = open(os.path.join(ref_root, "model", "DRT.py")).read()
    tree = ast.parse(src)
    wanted = {}
    for node in tree.body:
        if isinstance(node, ast.ClassDef) and node.name == "ChunkKVManager":
            wanted["ChunkKVManager"] = ast.get_source_segment(src, node)
        if isinstance(node, ast.ClassDef) and node.name == "DRT":
            for sub in node.body:
                if isinstance(sub, ast.FunctionDef) and sub.name in ("_enc_dec_score_mask", "_perform_batch_retrieval"):
                    wanted[sub.name] = textwrap.dedent(ast.get_source_segment(src, sub, padded=True))
        if isinstance(node, ast.ClassDef) and node.name == "TritonGroupCrossAttention":
            for sub in node.body:
                if isinstance(sub, ast.FunctionDef) and sub.name == "preprocess_chunk_kv_cache":
                    seg = textwrap.dedent(ast.get_source_segment(src, sub, padded=True))
                    wanted["preprocess_chunk_kv_cache"] = seg
    ns = dict(torch=torch, F=F, math=math, rearrange=rearrange, repeat=repeat)
    exec(wanted["ChunkKVManager"], ns)
    exec(wanted["preprocess_chunk_kv_cache"], ns)
    exec(wanted["_enc_dec_score_mask"], ns)
    exec(wanted["_perform_batch_retrieval"], ns)

    class DummyDRT:
        def __init__(self, input_dim, num_heads, chunk_topk, training=False):
            self.input_dim = input_dim
            self.num_heads = num_heads
            self.chunk_topk = chunk_topk
            self.training = training
            self.device = torch.device("cpu")
            self.causal_masks = {}
            self.preprocess_chunk_kv_cache = ns["preprocess_chunk_kv_cache"]
        _enc_dec_score_mask = ns["_enc_dec_score_mask"]
        _perform_batch_retrieval = ns["_perform_batch_retrieval"]

    decode_block = _slice_between(src, "past_lmk_embs = chunk_kvs.past_lmk_embeds  # (N, ?, dim)",
                                  "indices = indices.squeeze(1)")
    return ns["ChunkKVManager"], DummyDRT, decode_block


def module_case(seed: int, n: int, c: int, heads: int, k: int, dim: int):
    """Seeded inputs of the module fixtures: hidden (N, C, 64, dim), gathered chunks
    (N, (C-1)*K, 64, dim), weights (N, C-1, K), upstream gradient (N, C*64, dim), and the three
    parameter tensors."""
    g = torch.Generator().manual_seed(seed)
    hidden = torch.randn(n, c, 64, dim, generator=g)
    gk = torch.randn(n, (c - 1) * k, 64, dim, generator=g)
    gv = torch.randn(n, (c - 1) * k, 64, dim, generator=g)
    w = torch.softmax(torch.randn(n, c - 1, k, generator=g), -1)
    dout = torch.randn(n, c * 64, dim, generator=g)
    params = {"pre_norm.weight": 1.0 + 0.1 * torch.randn(dim, generator=g),
              "q_proj.weight": torch.randn(dim, dim, generator=g) / math.sqrt(dim),
              "o_proj.weight": torch.randn(dim, dim, generator=g) / math.sqrt(dim)}
    return hidden, gk, gv, w, dout, params


def lift_reference_modules(ref_root: str, einsum_block: str):
    """The reference's two GCA module classes, executable on CPU."""
    import torch.nn as nn
    src = open(os.path.join(ref_root, "model", "DRT.py")).read()
    tree = ast.parse(src)
    segs = {node.name: ast.get_source_segment(src, node) for node in tree.body
            if isinstance(node, ast.ClassDef) and node.name in ("TritonGroupCrossAttention", "GroupCrossAttention")}

    class RMSNorm(nn.Module):                     # stand-in for flash_attn.ops.rms_norm.RMSNorm: the plain formula
        def __init__(self, hidden_size, eps=1e-5):
            super().__init__()
            self.weight = nn.Parameter(torch.ones(hidden_size))
            self.eps = eps

        def forward(self, x):
            return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight

    def gca_einsum(q, k, v, weights, sm_scale, sm_n):     # the reference's einsum ground truth as the operator
        group = q.shape[1] // k.shape[1]
        ns_ = dict(torch=torch, q=q, k=k, v=v, weights=weights, sm_scale=sm_scale, dtype=q.dtype)
        exec(einsum_block.replace("repeats=4", f"repeats={group}"), ns_)
        return ns_["ref_out"]

    def flash_attn_func(q, k, v, causal=False):           # (B, S, h, d) plain softmax attention
        p = torch.softmax(torch.einsum('bqhd,bkhd->bhqk', q, k) / math.sqrt(q.shape[-1]), -1)
        return torch.einsum('bhqk,bkhd->bqhd', p, v)

    ns = dict(torch=torch, nn=nn, math=math, rearrange=rearrange, repeat=repeat, RMSNorm=RMSNorm, LlamaConfig=object,
              gca_attn=gca_einsum, gca_kv_cache=gca_einsum, flash_attn_func=flash_attn_func)
    exec(segs["GroupCrossAttention"], ns)
    exec(segs["TritonGroupCrossAttention"], ns)
    return ns["TritonGroupCrossAttention"], ns["GroupCrossAttention"]


def projection_case(seed: int):
    """Encoder outputs of an earlier append (1 chunk) and of the append under test (2 chunks), 2 sequences,
    256 wide, and the two projection matrices: all bf16-representable."""
    g = torch.Generator().manual_seed(seed)
    enc_prev = torch.randn(2, 1, 64, 256, generator=g).bfloat16().float()
    enc_new = torch.randn(2, 2, 64, 256, generator=g).bfloat16().float()
    wk = (torch.randn(256, 256, generator=g) / 16).bfloat16().float()
    wv = (torch.randn(256, 256, generator=g) / 16).bfloat16().float()
    return enc_prev, enc_new, wk, wv


class ModuleConfig:
    hidden_size, num_attention_heads, enc_chunk_size, chunk_topk = 128, 2, 63, 3
    rms_norm_eps, attention_bias, enable_softmax_one = 1e-5, False, False


def main(ref_root: str):
    torch.manual_seed(0)
    # ---- 1. GCA op: the reference's einsum ground truth, fp32 and its bf16 dtype path ----
    for name, (seed, z, hq, hkv, k, std, dtype, scale) in {
        "gca_ref_fp32_gqa4": (22, 2, 4, 1, 2, 0.5, torch.float32, 1 / 8),
        "gca_ref_fp32_mha": (0, 2, 2, 2, 4, 1.0, torch.float32, 1 / 8),
        "gca_ref_bf16_gqa4": (22, 2, 4, 1, 2, 0.5, torch.bfloat16, 1 / 8),
        "gca_ref_fp32_gqa2_scale05": (5, 2, 4, 2, 3, 0.5, torch.float32, 0.5),
    }.items():
        q, kk, v, w, dout = cases.gca_gathered_case(seed, z, hq, hkv, k, std=std, dtype=dtype)
        block = reference_einsum_block(ref_root, hq // hkv)
        o, dq, dk, dv, dw = run_reference_gca(block, q, kk, v, w, scale, dout, dtype)
        np.savez_compressed(os.path.join(HERE, name + ".npz"),
                            meta=np.array([seed, z, hq, hkv, k, std, scale], dtype=np.float64),
                            in_checksum=cases.checksum(q, kk, v, w, dout),
                            o=o.float().numpy(), dq=dq.float().numpy(), dk=dk.float().numpy(),
                            dv=dv.float().numpy(), dw=dw.float().numpy())
        print(name, "ok", float(o.float().abs().max()))

    # ---- 2. inference shapes of the reference test: q-len 2 and 1 (gca.py:967-1011) ----
    src = open(os.path.join(ref_root, "ltriton", "gca.py")).read()
    inf_block = _slice_between(src, "k_ = torch.repeat_interleave(k, dim=1, repeats=2)",
                               "ref_out = torch.einsum('Z H K M h, Z K->Z H M h', ref_out, weights)")
    for name, sq in (("gca_ref_inf_q2", 2), ("gca_ref_inf_q1", 1)):
        q, kk, v, w, _ = cases.gca_gathered_case(7 + sq, 3, 4, 2, 5, s=sq, std=0.5)
        ns = dict(torch=torch, q=q, k=kk, v=v, weights=w, sm_scale=0.5)
        exec(inf_block, ns)
        np.savez_compressed(os.path.join(HERE, name + ".npz"),
                            in_checksum=cases.checksum(q, kk, v, w), o=ns["ref_out"].numpy())
        print(name, "ok")

    # ---- 3. retrieval layer: the reference's own methods on CPU ----
    Manager, DummyDRT, decode_block = lift_reference_retrieval(ref_root)
    n, c, dmodel, heads, topk = 2, 12, 768, 12, 8
    lq, lk = cases.landmark_case(3, n, c, c, d=dmodel)
    g = torch.Generator().manual_seed(4)
    chunk_k = torch.randn(n, c, 64, dmodel, generator=g)
    chunk_v = torch.randn(n, c, 64, dmodel, generator=g)
    mgr = Manager(False, 1)
    mgr.append(chunk_k[:, :5], chunk_v[:, :5], lk[:, :5].float())
    mgr.append(chunk_k[:, 5:], chunk_v[:, 5:], lk[:, 5:].float())      # growth by torch.cat
    drt = DummyDRT(dmodel, heads, topk, training=False)
    ck, cv, cw, indices = drt._perform_batch_retrieval(lq.float(), mgr, 0, use_cache=True)
    cur_k, cur_v, cur_w = mgr.current_retrieved_chunk(0)
    scores = torch.einsum('ncd,ned->nce', lq.float(), lk.float()) / math.sqrt(dmodel)
    np.savez_compressed(os.path.join(HERE, "retrieval_ref_batch.npz"),
                        in_checksum=cases.checksum(lq, lk, chunk_k, chunk_v),
                        indices=indices.numpy(), weights=cw.numpy(), scores=scores.numpy(),
                        chunk_k_shape=np.array(ck.shape), chunk_k_sum=ck.double().sum(dim=(-1, -2)).numpy(),
                        chunk_v_sum=cv.double().sum(dim=(-1, -2)).numpy(),
                        cur_k_sum=cur_k.double().sum(dim=(-1, -2)).numpy(), cur_w=cur_w.numpy())
    print("retrieval_ref_batch ok", tuple(ck.shape), tuple(indices.shape))

    # decode-time retrieval statements (DRT.py:836-845), executed with the names they use
    class SelfNS:
        input_dim = dmodel
        chunk_topk = topk
    selfns = DummyDRT(dmodel, heads, topk)
    g = torch.Generator().manual_seed(9)
    hidden_states = torch.randn(n, 2, dmodel, generator=g).bfloat16().float()
    ns = dict(torch=torch, F=F, math=math, chunk_kvs=mgr, hidden_states=hidden_states, self=selfns)
    exec(decode_block, ns)
    np.savez_compressed(os.path.join(HERE, "retrieval_ref_decode.npz"),
                        in_checksum=cases.checksum(hidden_states, lk),
                        indices=ns["indices"].numpy(), weights=ns["weights"].numpy())
    print("retrieval_ref_decode ok", tuple(ns["indices"].shape))

    # ---- 5. the GCA sub-layer modules (DRT.py:235-398), forward + backward, train and eval mode ----
    src_gca = open(os.path.join(ref_root, "ltriton", "gca.py")).read()
    einsum_block = _slice_between(src_gca, "k_ = torch.repeat_interleave(k, dim=1, repeats=4)",
                                  "ref_out = torch.einsum('Z H K M h, Z K->Z H M h', o_k, weights)")
    TritonMod, FlashMod = lift_reference_modules(ref_root, einsum_block)
    cfg = ModuleConfig()
    n_, c_, k_ = 1, 3, cfg.chunk_topk
    hidden, gk, gv, w, dout, params = module_case(51, n_, c_, cfg.num_attention_heads, k_, cfg.hidden_size)
    out = {"in_checksum": cases.checksum(hidden, gk, gv, w, dout, *params.values())}
    for tag, cls in (("triton", TritonMod), ("flash", FlashMod)):
        mod = cls(cfg)
        mod.load_state_dict(params)
        ck, cv, cw = cls.preprocess_chunk_kv_cache(gk, gv, w, cfg.num_attention_heads)
        for mode in ("train", "eval"):
            mod.train(mode == "train")
            mod.zero_grad()
            hs = hidden.clone().requires_grad_()
            o = mod(hs, ck, cv, cw)
            o.backward(dout)
            out[f"{tag}_{mode}_o"] = o.detach().numpy()
            if mode == "train":
                out[f"{tag}_dhidden"] = hs.grad.numpy()
                out[f"{tag}_dq_proj"] = mod.q_proj.weight.grad.numpy().copy()
                out[f"{tag}_do_proj"] = mod.o_proj.weight.grad.numpy().copy()
        # decode step: one chunk, one row (D = 1, S = 1): no first-chunk padding
        mod.eval()
        with torch.no_grad():
            o1 = mod(hidden[:, 1:2, :1], *cls.preprocess_chunk_kv_cache(gk[:, :k_], gv[:, :k_], w[:, :1], cfg.num_attention_heads))
        out[f"{tag}_decode_o"] = o1.numpy()
    np.savez_compressed(os.path.join(HERE, "module_ref.npz"), **out)
    print("module_ref ok", {k2: v2.shape for k2, v2 in out.items() if hasattr(v2, "shape") and v2.ndim > 0 and "train_o" in k2})

    # ---- 6. chunk K/V projection + landmark clearing + append (DRT.py:766-784), after an earlier append ----
    import torch.nn as nn
    src_drt = open(os.path.join(ref_root, "model", "DRT.py")).read()
    proj_block = _slice_between(src_drt, "lmk_embs = chunk_hidden_states[:, :, -1, :]", "chunk_kvs.append(chunk_k, chunk_v, lmk_embs)")
    enc_prev, enc_new, wk, wv = projection_case(61)

    class ProjSelf:
        chunk_k_proj = nn.Linear(256, 256, bias=False)
        chunk_v_proj = nn.Linear(256, 256, bias=False)
    with torch.no_grad():
        ProjSelf.chunk_k_proj.weight.copy_(wk)
        ProjSelf.chunk_v_proj.weight.copy_(wv)
        mgr6 = Manager(False, 1)
        for enc in (enc_prev, enc_new):
            exec(proj_block, dict(torch=torch, self=ProjSelf, chunk_hidden_states=enc.clone(), chunk_kvs=mgr6))
    np.savez_compressed(os.path.join(HERE, "projection_ref.npz"), in_checksum=cases.checksum(enc_prev, enc_new, wk, wv),
                        chunk_k=mgr6.chunk_k.numpy().astype(np.float16), chunk_v=mgr6.chunk_v.numpy().astype(np.float16),
                        lmk=mgr6.past_lmk_embeds.numpy())
    print("projection_ref ok", tuple(mgr6.chunk_k.shape))

    # ---- 4. mask (DRT.py:590-607) for a few shapes ----
    masks = {}
    for cq, e in ((1, 1), (1, 9), (4, 4), (3, 10), (12, 12)):
        masks[f"mask_{cq}_{e}"] = drt._enc_dec_score_mask(cq, e).numpy()
    np.savez_compressed(os.path.join(HERE, "retrieval_ref_masks.npz"), **masks)
    print("masks ok")


if __name__ == "__main__":
    # the reference checkout: argument, else $GCA_REFERENCE, else a `reference` directory beside this repository
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("GCA_REFERENCE") or
         os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"))
