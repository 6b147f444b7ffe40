"""The GCA sub-layer modules against the REFERENCE's own module classes.

``tests/golden/make_golden.py`` lifts ``TritonGroupCrossAttention`` and ``GroupCrossAttention``
(``model/DRT.py:235-398``) out of the reference checkout by source text and runs them on CPU with
stand-ins for their three third-party callables; ``module_ref.npz`` holds their outputs and
gradients.  Here this repository's modules load the same parameters, get the same seeded
inputs, and must reproduce output, input gradient and both projection gradients: that pins the
glue around the operator (norm, projection, head split, first chunk dropped and zero-filled,
the flash variant's layout, the output projection), in train mode, eval mode and for a
one-row decode step.  float32 end to end (the CUDA-core kernels): 1e-4.
"""
import os

import numpy as np
import pytest
import torch

import cases
import make_golden as MG

pytestmark = pytest.mark.gpu


def rel(a, b):
    a, b = a.detach().float().cpu(), torch.as_tensor(b).float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


@pytest.mark.parametrize("tag", ["triton", "flash"])
def test_module_matches_reference_class(golden_dir, tag):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import long_context_modeling_b200 as lcm
    g = np.load(os.path.join(golden_dir, "module_ref.npz"))
    cfg = MG.ModuleConfig()
    n, c, k = 1, 3, cfg.chunk_topk
    hidden, gk, gv, w, dout, params = MG.module_case(51, n, c, cfg.num_attention_heads, k, cfg.hidden_size)
    assert abs(cases.checksum(hidden, gk, gv, w, dout, *params.values()) - float(g["in_checksum"])) < 1e-6
    cls = lcm.TritonGroupCrossAttention if tag == "triton" else lcm.GroupCrossAttention
    mod = cls(cfg).cuda()                                   # constructed from a config object, like the reference
    mod.load_state_dict({k_: v_.cuda() for k_, v_ in params.items()})
    ck, cv, cw = cls.preprocess_chunk_kv_cache(gk.cuda(), gv.cuda(), w.cuda(), cfg.num_attention_heads)
    for mode in ("train", "eval"):
        mod.train(mode == "train")
        mod.zero_grad()
        hs = hidden.cuda().requires_grad_()
        o = mod(hs, ck, cv, cw)
        assert o.shape == g[f"{tag}_{mode}_o"].shape
        assert rel(o, g[f"{tag}_{mode}_o"]) <= 1e-4, mode
        assert o[:, :64].abs().max().item() == 0            # the first chunk retrieves nothing
        if mode == "train":
            o.backward(dout.cuda())
            assert rel(hs.grad, g[f"{tag}_dhidden"]) <= 1e-4
            assert rel(mod.q_proj.weight.grad, g[f"{tag}_dq_proj"]) <= 1e-4
            assert rel(mod.o_proj.weight.grad, g[f"{tag}_do_proj"]) <= 1e-4
    mod.eval()
    with torch.no_grad():
        o1 = mod(hidden[:, 1:2, :1].cuda(), *cls.preprocess_chunk_kv_cache(gk[:, :k].cuda(), gv[:, :k].cuda(), w[:, :1].cuda(),
                                                                         cfg.num_attention_heads))
    assert rel(o1, g[f"{tag}_decode_o"]) <= 1e-4


def test_manager_keeps_the_autograd_graph_through_append_retrieve_and_gca():
    """Training route through ``ChunkKVManager``: the chunk K/V and landmark tensors handed to
    ``append`` come out of projections; gradients must reach them through
    ``gca_indexed(..., mgr.chunk_k, mgr.chunk_v, ...)`` and through the retrieval weights
    (``model/DRT.py:87-133,626,784``).  Reference: the same composition in plain torch autograd
    (gather + einsum GCA + softmax of the gathered scores) in float64."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import long_context_modeling_b200 as lcm
    from oracle import gca_oracle as G
    dev = "cuda"
    n, c, h, k, dim = 2, 7, 2, 3, 128
    g = torch.Generator().manual_seed(77)
    x = torch.randn(n, c, 64, dim, generator=g)
    wk = torch.randn(dim, dim, generator=g) / dim ** 0.5
    wv = torch.randn(dim, dim, generator=g) / dim ** 0.5
    wl = torch.randn(dim, dim, generator=g) / dim ** 0.5
    q = torch.randn(n, c - 1, h, 64, 64, generator=g)
    lq = torch.randn(n, c, dim, generator=g).bfloat16().float()
    dout = torch.randn(n, c - 1, h, 64, 64, generator=g)

    def forward(use_lib: bool, dtype, device):
        xs = x.to(device, dtype)
        pk, pv, pl, lqp = (t.to(device, dtype).requires_grad_() for t in (wk, wv, wl, lq))
        chunk_k, chunk_v = xs @ pk, xs @ pv
        lmk = xs[:, :, -1] @ pl
        if use_lib:
            mgr = lcm.ChunkKVManager()
            mgr.append(chunk_k, chunk_v, lmk)
            assert mgr.tracks_gradients and mgr.chunk_k.requires_grad
            idx, wts, _ = lcm.retrieve(lqp, mgr, k, training=False)
            out = lcm.gca_indexed(q.to(device, dtype), mgr.chunk_k, mgr.chunk_v, idx, wts, 0.125)
            res_idx = idx
        else:
            idx_full = forward.idx                      # same selection as the library run
            wts = lcm.differentiable_weights(lqp, lmk, idx_full.to(device))[:, :-1]
            out = G.gca_indexed(q.to(device, dtype), chunk_k, chunk_v, idx_full[:, :-1].to(device), wts, 0.125)
            res_idx = None
        out.backward(dout.to(device, dtype))
        return out.detach(), pk.grad, pv.grad, pl.grad, lqp.grad, res_idx

    got = forward(True, torch.float32, dev)
    # the full-row indices of the library run (row i serves query chunk i + 1; the last row is dropped)
    mgr2 = lcm.ChunkKVManager()
    with torch.no_grad():
        xs = x.to(dev)
        mgr2.append(xs @ wk.to(dev), xs @ wv.to(dev), xs[:, :, -1] @ wl.to(dev))
        forward.idx = lcm.lmk_score_topk(lq.to(dev), mgr2.past_lmk_embeds, k).indices.cpu()
    assert not mgr2.tracks_gradients                    # appended under no_grad: the in-place buffer path
    assert torch.equal(forward.idx[:, :-1], got[5].cpu())
    ref = forward(False, torch.float64, "cpu")
    for name, a, b in zip(("out", "d chunk_k_proj", "d chunk_v_proj", "d landmark proj", "d query landmarks"), got[:5], ref[:5]):
        assert a is not None, name
        err = ((a.double().cpu() - b).abs().max() / (b.abs().max() + 1e-12)).item()
        # landmarks are scored in bf16 by the scan but re-scored differentiably in the input dtype
        assert err <= (5e-3 if "landmark" in name else 1e-4), (name, err)
