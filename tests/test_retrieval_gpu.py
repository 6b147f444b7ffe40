"""Landmark scoring / top-k / cache on the GPU against the canonical CPU oracle and the
golden vectors produced by the reference's own retrieval code.  Indices must match
BIT-EXACTLY (ties to the lower chunk id); weights and scores within float32 rounding.
"""
import math
import os

import numpy as np
import pytest
import torch

import cases
from oracle import retrieval_oracle as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lcm():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import long_context_modeling_b200 as m
    return m


def oracle_rows(lq, lk, topk, q_pos0=None, e_base=0, noise=None, head_dim=0, score_round="fp32"):
    """Per-sequence oracle over a batch: returns idx (N, Cq[, H], K), weights, scores, nvalid."""
    n, cq, d = lq.shape
    e = lk.shape[1]
    q_pos0 = (e - cq) if q_pos0 is None else q_pos0
    limit = q_pos0 + np.arange(cq)
    out = []
    for b in range(n):
        s = R.canonical_scores(lq[b].float().numpy(), lk[b].float().numpy(), head_dim=head_dim, score_round=score_round)
        if head_dim:
            per_head = [R.canonical_topk(s[:, hh, :], limit, topk, e_base=e_base) for hh in range(s.shape[1])]
            out.append(tuple(np.stack([ph[i] for ph in per_head], axis=1) for i in range(4)))
        else:
            nz = None if noise is None else noise[b].numpy()
            out.append(R.canonical_topk(s, limit, topk, noise=nz, e_base=e_base))
    return tuple(np.stack([o[i] for o in out]) for i in range(4))


def check(res, ref, exact_scores=True):
    idx, clean, w, nv = ref
    assert np.array_equal(res.indices.cpu().numpy(), idx), "indices must be bit-exact"
    assert np.array_equal(res.n_valid.cpu().numpy(), nv)
    got_s = res.scores.cpu().numpy()
    fin = np.isfinite(clean)
    if exact_scores:
        assert np.array_equal(got_s[fin].view(np.uint32), clean[fin].view(np.uint32)), "scores must be bit-exact"
    assert np.all(np.isneginf(got_s[~fin]))
    assert np.allclose(res.weights.cpu().numpy(), w, atol=2e-6)


@pytest.mark.parametrize("n,cq,e,d,k", [(2, 12, 12, 768, 8), (1, 260, 260, 768, 8), (3, 5, 37, 128, 4),
                                         (2, 1, 300, 768, 8), (1, 7, 7, 256, 32), (2, 3, 1000, 512, 16)])
def test_topk_bit_exact_vs_canonical_oracle(lcm, n, cq, e, d, k):
    lq, lk = cases.landmark_case(21, n, cq, e, d=d)
    res = lcm.lmk_score_topk(lq.cuda(), lk.cuda(), k)
    check(res, oracle_rows(lq, lk, k))


def test_topk_matches_reference_golden(lcm, golden_dir):
    """Indices / weights produced by the reference's ``_perform_batch_retrieval`` and its
    decode-time block, run from the reference source on CPU."""
    g = np.load(os.path.join(golden_dir, "retrieval_ref_batch.npz"))
    n, c, d, topk = 2, 12, 768, 8
    lq, lk = cases.landmark_case(3, n, c, c, d=d)
    res = lcm.lmk_score_topk(lq.cuda(), lk.cuda(), topk)
    idx = res.indices.cpu().numpy()
    w = res.weights.cpu().numpy()
    ref_w = g["weights"].reshape(n, c - 1, topk)
    for b in range(n):
        for i in range(c - 1):
            m = min(i, topk)
            assert np.array_equal(idx[b, i, :m], g["indices"][b, i, :m])
            assert np.allclose(w[b, i, :m], ref_w[b, i, :m], atol=1e-5)
            assert np.all(idx[b, i, m:] == -1) and np.all(w[b, i, m:] == 0)
    gd = np.load(os.path.join(golden_dir, "retrieval_ref_decode.npz"))
    hidden = torch.randn(n, 2, d, generator=torch.Generator().manual_seed(9)).bfloat16()
    res = lcm.lmk_score_topk(hidden[:, -1:].cuda(), lk.cuda(), topk)
    assert np.array_equal(res.indices.cpu().numpy()[:, 0], gd["indices"])
    assert np.allclose(res.weights.cpu().numpy(), gd["weights"], atol=1e-5)


def test_ties_masked_rows_and_all_masked(lcm):
    g = torch.Generator().manual_seed(2)
    lk = torch.randn(1, 50, 768, generator=g).bfloat16()
    lk[0, 31] = lk[0, 4]
    lk[0, 17] = lk[0, 4]                      # three identical landmarks: exact ties
    lq = (lk[:, 4:5] * 3).bfloat16()
    res = lcm.lmk_score_topk(lq.cuda(), lk.cuda(), 8, q_pos0=50)
    assert res.indices[0, 0, :3].tolist() == [4, 17, 31]
    check(res, oracle_rows(lq, lk, 8, q_pos0=50))
    # fewer visible chunks than K, and a row that sees nothing
    lq3 = torch.randn(1, 3, 768, generator=g).bfloat16()
    res = lcm.lmk_score_topk(lq3.cuda(), lk.cuda(), 8, q_pos0=0)    # rows see 0, 1, 2 chunks
    assert res.n_valid[0].tolist() == [0, 1, 2]
    assert torch.all(res.weights[0, 0] == 0) and torch.all(res.indices[0, 0] == -1)
    check(res, oracle_rows(lq3, lk, 8, q_pos0=0))


@pytest.mark.parametrize("splits", [1, 2, 7, 40])
def test_result_independent_of_split_count(lcm, splits):
    lq, lk = cases.landmark_case(22, 2, 2, 5000, d=768)
    base = lcm.lmk_score_topk(lq.cuda(), lk.cuda(), 8, splits=1)
    res = lcm.lmk_score_topk(lq.cuda(), lk.cuda(), 8, splits=splits)
    assert torch.equal(res.keys, base.keys) and torch.equal(res.indices, base.indices)
    check(res, oracle_rows(lq, lk, 8))


def test_per_head_mode(lcm):
    lq, lk = cases.landmark_case(23, 2, 1, 3000, d=768, std=0.125)
    res = lcm.lmk_score_topk(lq.cuda(), lk.cuda(), 8, head_dim=64)
    assert res.indices.shape == (2, 1, 12, 8)
    check(res, oracle_rows(lq, lk, 8, head_dim=64))


def test_noise_selects_but_weights_stay_noise_free(lcm):
    """Training: Gumbel noise perturbs the selection only (DRT.py:616-626)."""
    n, c, d, k = 2, 20, 768, 4
    lq, lk = cases.landmark_case(24, n, c, c, d=d)
    noise = -torch.empty(n, c, c).exponential_(generator=torch.Generator().manual_seed(3)).log()
    res = lcm.lmk_score_topk(lq.cuda(), lk.cuda(), k, noise=noise.cuda())
    check(res, oracle_rows(lq, lk, k, noise=noise))
    plain = lcm.lmk_score_topk(lq.cuda(), lk.cuda(), k)
    assert not torch.equal(plain.indices, res.indices)


def test_bf16_score_rounding_mode(lcm):
    lq, lk = cases.landmark_case(25, 1, 2, 4000, d=768)
    res = lcm.lmk_score_topk(lq.cuda(), lk.cuda(), 8, score_round="bf16")
    check(res, oracle_rows(lq, lk, 8, score_round="bf16"))


def test_set_equality_with_torch_topk(lcm):
    lq, lk = cases.landmark_case(26, 2, 6, 500, d=768)
    res = lcm.lmk_score_topk(lq.cuda(), lk.cuda(), 8)
    ti, tw = R.torch_reference_retrieval(lq.float(), lk.float(), 8)
    for b in range(2):
        for i in range(6):
            assert set(res.indices[b, i].tolist()) == set(ti[b, i].tolist())
    assert np.allclose(np.sort(res.weights.cpu().numpy(), -1), np.sort(tw.numpy(), -1), atol=1e-5)


def test_merge_of_shards_equals_single_scan(lcm):
    """Chunk-range sharding: local top-k per shard (global ids) + merge == one scan."""
    lq, lk = cases.landmark_case(27, 1, 1, 8192, d=768)
    full = lcm.lmk_score_topk(lq.cuda(), lk.cuda(), 8)
    for shards in (2, 4, 8):
        per = 8192 // shards
        parts = [lcm.lmk_score_topk(lq.cuda(), lk[:, r * per:(r + 1) * per].contiguous().cuda(), 8,
                                    q_pos0=8191, e_base=r * per).keys for r in range(shards)]
        merged = lcm.merge_topk(torch.cat(parts, dim=-1), 8)
        assert torch.equal(merged.keys, full.keys)
        assert torch.equal(merged.indices, full.indices)
        assert torch.allclose(merged.weights, full.weights, atol=1e-6)
        ref = R.merge_candidates(torch.cat(parts, -1).cpu().numpy().view(np.uint64).reshape(1, -1), 8)
        assert np.array_equal(merged.keys.cpu().numpy().view(np.uint64).reshape(1, -1), ref)


def test_full_size_16m_token_landmark_scan(lcm):
    """BASELINE retrieval config: 262,144 landmarks x 768 (bf16), one query, top-8 per head
    and per sequence.  Checked against the oracle on the winners' neighbourhood: every
    selected score must be the canonical score of that chunk, sorted, and no unselected
    chunk of a random sample may beat the 8th."""
    e, d = 262144, 768
    g = torch.Generator().manual_seed(0)
    lk = (torch.randn(e, d, generator=g) * 0.125).bfloat16()
    lq = (torch.randn(1, d, generator=g) * 0.125).bfloat16()
    for head_dim in (0, 64):
        res = lcm.lmk_score_topk(lq[None].cuda(), lk[None].cuda(), 8, head_dim=head_dim)
        idx = res.indices.cpu().numpy().reshape(-1, 8)
        sc = res.scores.cpu().numpy().reshape(-1, 8)
        sample = np.unique(np.concatenate([idx.reshape(-1), np.random.default_rng(0).integers(0, e - 1, 4096)]))
        s = R.canonical_scores(lq.float().numpy(), lk[sample].float().numpy(), head_dim=head_dim).reshape(-1, len(sample))
        pos = {int(v): i for i, v in enumerate(sample)}
        for r in range(idx.shape[0]):
            assert np.all(idx[r] < e - 1)                      # the newest chunk is never visible
            mine = np.array([s[r, pos[int(i)]] for i in idx[r]], dtype=np.float32)
            assert np.array_equal(mine.view(np.uint32), sc[r].view(np.uint32))
            assert np.all(np.diff(sc[r]) <= 0)
            others = np.delete(s[r], [pos[int(i)] for i in idx[r]])
            assert others.max() <= sc[r, -1]
    # whole-scan equality against float64 argsort on a tie-free instance
    full = (lk.double() @ lq[0].double()).numpy() / math.sqrt(d)
    full[-1] = -np.inf
    top = np.argsort(-full, kind="stable")[:8]
    res = lcm.lmk_score_topk(lq[None].cuda(), lk[None].cuda(), 8)
    assert set(res.indices.cpu().numpy().reshape(-1).tolist()) == set(top.tolist())


def test_chunk_cache_manager_and_drop_in_retrieval(lcm, golden_dir):
    """ChunkKVManager mirror + perform_batch_retrieval against the reference's own outputs."""
    g = np.load(os.path.join(golden_dir, "retrieval_ref_batch.npz"))
    n, c, dmodel, heads, topk = 2, 12, 768, 12, 8
    lq, lk = cases.landmark_case(3, n, c, c, d=dmodel)
    gen = torch.Generator().manual_seed(4)
    chunk_k = torch.randn(n, c, 64, dmodel, generator=gen)
    chunk_v = torch.randn(n, c, 64, dmodel, generator=gen)
    mgr = lcm.ChunkKVManager(False, 1)
    mgr.append(chunk_k[:, :5].cuda(), chunk_v[:, :5].cuda(), lk[:, :5].float().cuda())
    mgr.append(chunk_k[:, 5:].cuda(), chunk_v[:, 5:].cuda(), lk[:, 5:].float().cuda())   # growth
    assert len(mgr) == c and torch.equal(mgr.chunk_k.cpu(), chunk_k) and torch.equal(mgr.chunk_v.cpu(), chunk_v)
    assert torch.equal(mgr.past_lmk_embeds.cpu(), lk.float())
    ck, cv, cw, indices = lcm.perform_batch_retrieval(lq.float().cuda(), mgr, 0, num_heads=heads, chunk_topk=topk,
                                                      use_cache=True)
    assert tuple(ck.shape) == tuple(g["chunk_k_shape"]) and indices.dtype == torch.int64
    ref_w = g["weights"]
    assert np.allclose(cw.cpu().numpy(), ref_w, atol=1e-5)
    # gathered tensors: compare per-(row, head, slot) sums where the weight is non-zero
    live = (ref_w > 0)[:, None, :]
    ks = ck.double().sum(dim=(-1, -2)).cpu().numpy()
    vs = cv.double().sum(dim=(-1, -2)).cpu().numpy()
    assert np.allclose(np.where(live, ks, 0), np.where(live, g["chunk_k_sum"], 0), atol=1e-6)
    assert np.allclose(np.where(live, vs, 0), np.where(live, g["chunk_v_sum"], 0), atol=1e-6)
    cur_k, cur_v, cur_w = mgr.current_retrieved_chunk(0)
    assert np.allclose(cur_w.cpu().numpy(), g["cur_w"], atol=1e-5)
    assert np.allclose(cur_k.double().sum(dim=(-1, -2)).cpu().numpy(), g["cur_k_sum"], atol=1e-6)
    # zero-landmark append variant (DRT.py:771-781 folded into the append kernel)
    mgr2 = lcm.ChunkKVManager(zero_landmark=True, capacity=64)
    mgr2.append(chunk_k.cuda().bfloat16(), chunk_v.cuda().bfloat16(), lk.cuda())
    assert mgr2.chunk_k[:, :, -1].abs().max().item() == 0 and mgr2.chunk_v[:, :, -1].abs().max().item() == 0
    assert torch.equal(mgr2.chunk_k[:, :, :-1].cpu(), chunk_k.bfloat16()[:, :, :-1])


def test_differentiable_weights_match_reference_autograd(lcm):
    """Gradients of the retrieval weights w.r.t. the landmarks equal autograd through the
    reference sequence softmax(scores.gather(topk)) (DRT.py:612-626)."""
    n, c, d, k = 2, 9, 768, 4
    lq, lk = cases.landmark_case(28, n, c, c, d=d)
    lqg = lq.float().cuda().requires_grad_()
    lkg = lk.float().cuda().requires_grad_()
    res = lcm.lmk_score_topk(lqg, lkg, k)
    w = lcm.differentiable_weights(lqg, lkg, res.indices)
    probe = torch.randn(w.shape, generator=torch.Generator().manual_seed(1)).cuda()
    (w * probe).sum().backward()
    a = lq.float().requires_grad_()
    b = lk.float().requires_grad_()
    ti, tw = R.torch_reference_retrieval(a, b, k)
    # align slots: the reference orders by score too; padding differs only where weight is 0
    (tw * probe.cpu()).sum().backward()
    assert torch.allclose(w.detach().cpu(), tw.detach(), atol=1e-5)
    assert torch.allclose(lqg.grad.cpu(), a.grad, atol=1e-4)
    assert torch.allclose(lkg.grad.cpu(), b.grad, atol=1e-4)


def test_projection_with_append_epilogue_matches_reference_statements(lcm, golden_dir):
    """``ChunkKVManager.append_projected`` (one tensor-core GEMM whose epilogue writes K and V into the
    cache, landmark rows cleared, landmark embeddings extracted) against the reference's own statements
    ``model/DRT.py:766-784`` run on the reference's own manager, for an append that follows an earlier
    one (non-zero position, cache growth)."""
    import make_golden as MG
    g = np.load(os.path.join(golden_dir, "projection_ref.npz"))
    enc_prev, enc_new, wk, wv = MG.projection_case(61)
    assert abs(cases.checksum(enc_prev, enc_new, wk, wv) - float(g["in_checksum"])) < 1e-6
    mgr = lcm.ChunkKVManager(zero_landmark=True, capacity=2)          # capacity 2 < 3 chunks: the buffer also grows
    wk_d, wv_d = wk.cuda().bfloat16(), wv.cuda().bfloat16()
    with torch.no_grad():
        for enc in (enc_prev, enc_new):
            mgr.append_projected(enc.cuda().bfloat16(), wk_d, wv_d)
    torch.cuda.synchronize()
    assert lcm.read_status() == 0 and len(mgr) == 3 and not mgr.tracks_gradients
    for name, got in (("chunk_k", mgr.chunk_k), ("chunk_v", mgr.chunk_v), ("lmk", mgr.past_lmk_embeds)):
        ref = torch.from_numpy(g[name].astype(np.float32))
        assert got.shape == ref.shape, name
        err = (got.float().cpu() - ref).abs().max().item() / (ref.abs().max().item() + 1e-12)
        assert err <= 1e-2, (name, err)
    assert mgr.chunk_k[:, :, -1].abs().max().item() == 0 and mgr.chunk_v[:, :, -1].abs().max().item() == 0
    # more row tiles than CTAs, and a row count that is not a multiple of the 128-row tile
    gen = torch.Generator().manual_seed(62)
    enc = torch.randn(3, 101, 64, 256, generator=gen).bfloat16()
    big = lcm.ChunkKVManager(zero_landmark=False)
    with torch.no_grad():
        big.append_projected(enc.cuda(), wk_d, wv_d)
    want_k = (enc.float() @ wk.t())
    err = (big.chunk_k.float().cpu() - want_k).abs().max().item() / want_k.abs().max().item()
    assert err <= 1e-2, err
    assert lcm.read_status() == 0


def test_virtual_memory_cache_grows_in_place():
    """``ChunkKVManager(max_chunks=...)``: K and V sit in a virtual-address reservation, memory is mapped
    behind it as the cache fills.  Same contents as the doubling buffer after every append (plain and
    projected), addresses never change, the kernels read it like any cache, the reservation's limit is
    enforced, and the memory comes back on close()."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import long_context_modeling_b200 as lcm
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(21)
    n, l, hd = 3, 64, 256                                    # 32 KB per chunk: a 2 MB page holds 64 of them
    virt = lcm.ChunkKVManager(zero_landmark=True, max_chunks=200, capacity=16)
    plain = lcm.ChunkKVManager(zero_landmark=True)
    free0 = torch.cuda.mem_get_info(dev)[0]
    ptr = None
    wk = (torch.randn(hd, hd, generator=g) / 16).bfloat16().to(dev)
    wv = (torch.randn(hd, hd, generator=g) / 16).bfloat16().to(dev)
    for step in range(7):
        count = 23 + step
        if step % 2 == 0:
            k = torch.randn(n, count, l, hd, generator=g).bfloat16().to(dev)
            v = torch.randn(n, count, l, hd, generator=g).bfloat16().to(dev)
            lm = torch.randn(n, count, hd, generator=g).bfloat16().to(dev)
            virt.append(k, v, lm)
            plain.append(k, v, lm)
        else:
            x = torch.randn(n, count, l, hd, generator=g).bfloat16().to(dev)
            virt.append_projected(x, wk, wv)
            plain.append_projected(x, wk, wv)
        assert len(virt) == len(plain)
        assert torch.equal(virt.chunk_k, plain.chunk_k) and torch.equal(virt.chunk_v, plain.chunk_v)
        assert torch.equal(virt.past_lmk_embeds, plain.past_lmk_embeds)
        if ptr is None:
            ptr = virt.chunk_k.data_ptr()
        assert virt.chunk_k.data_ptr() == ptr                # grown in place
    c = len(virt)
    assert c == sum(23 + s for s in range(7)) and c <= 200
    # the kernels read the virtual cache like any other: retrieval + indexed GCA
    q = torch.randn(n, 1, 4, 1, 64, generator=g).bfloat16().to(dev)
    lq = torch.randn(n, 1, hd, generator=g).bfloat16().to(dev)
    r = lcm.lmk_score_topk(lq, virt.past_lmk_embeds, 8)
    rp = lcm.lmk_score_topk(lq, plain.past_lmk_embeds, 8)
    assert torch.equal(r.indices, rp.indices)
    o = lcm.gca_indexed_nograd(q, virt.chunk_k, virt.chunk_v, r.indices, r.weights, 0.125)
    op = lcm.gca_indexed_nograd(q, plain.chunk_k, plain.chunk_v, rp.indices, rp.weights, 0.125)
    assert torch.equal(o, op)
    with pytest.raises(ValueError):                           # beyond the reservation
        virt.append(torch.zeros(n, 60, l, hd, dtype=torch.bfloat16, device=dev), torch.zeros(n, 60, l, hd, dtype=torch.bfloat16, device=dev),
                    torch.zeros(n, 60, hd, dtype=torch.bfloat16, device=dev))
    torch.cuda.synchronize()
    used = free0 - torch.cuda.mem_get_info(dev)[0]
    del o, r
    virt.close()
    assert len(virt) == 0
    assert torch.cuda.mem_get_info(dev)[0] > free0 - used + 2 * n * (1 << 21)        # the mapped pages were released
