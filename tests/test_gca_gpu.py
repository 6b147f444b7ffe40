"""GCA parity on the GPU: the CUDA kernels (through the Python host layer and the C ABI)
against the CPU oracle and against the golden vectors produced by the reference's source.

Tolerances: bf16 -- 2e-2 relative to the largest reference magnitude (the north-star
bound) and the reference test's own ``atol=1e-2`` on out/dq/dk/dv, ``0.5`` on dw
(``ltriton/gca.py:938-961``); fp32 -- 1e-4 relative.
"""
import os

import numpy as np
import pytest
import torch

import cases
from oracle import gca_oracle as G

pytestmark = pytest.mark.gpu

BF16_REL, FP32_REL = 2e-2, 1e-4


@pytest.fixture(scope="module")
def lcm():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import long_context_modeling_b200 as m
    return m


def rel(a, b):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


def run_indexed(lcm, q, kc, vc, idx, w, scale, dout=None, algo=0, **kw):
    dev = "cuda"
    qd = q.to(dev).requires_grad_(dout is not None)
    kd = kc.to(dev).requires_grad_(dout is not None)
    vd = vc.to(dev).requires_grad_(dout is not None)
    wd = w.to(dev).requires_grad_(dout is not None)
    o = lcm.gca_indexed(qd, kd, vd, idx.to(dev), wd, scale, algo=algo, **kw)
    if dout is None:
        return o
    o.backward(dout.to(dev))
    return o, qd.grad, kd.grad, vd.grad, wd.grad


ALGOS = [pytest.param(1, id="cudacore"), pytest.param(2, id="tensorcore")]


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("n,c,h,k", [(2, 12, 4, 4), (1, 20, 12, 8), (2, 6, 3, 2)])
def test_fwd_bf16_vs_oracle(lcm, algo, n, c, h, k):
    q, kc, vc, idx, w, _ = cases.gca_indexed_case(0, n, c, h, k, dtype=torch.bfloat16)
    ref = G.gca_indexed(q.float(), kc.float(), vc.float(), idx, w, 0.125)
    out = run_indexed(lcm, q, kc, vc, idx, w, 0.125, algo=algo)
    assert out.dtype == torch.bfloat16 and out.shape == ref.shape
    assert rel(out, ref) <= BF16_REL
    assert (out.float().cpu() - ref).abs().max().item() <= 1e-2 * max(1.0, ref.abs().max().item())
    assert lcm.read_status() == 0
    # first query chunk retrieves nothing: exact zeros
    assert out[:, 0].abs().max().item() == 0.0


@pytest.mark.parametrize("n,c,h,k", [(2, 12, 4, 4), (1, 9, 2, 8)])
def test_fwd_bwd_fp32_vs_oracle(lcm, n, c, h, k):
    q, kc, vc, idx, w, dout = cases.gca_indexed_case(1, n, c, h, k, dtype=torch.float32)
    ref = G.gca_indexed_grads(q, kc, vc, idx, w, 0.125, dout, work_dtype=torch.float64)
    got = run_indexed(lcm, q, kc, vc, idx, w, 0.125, dout=dout)
    for name, g_, r_ in zip(("o", "dq", "dk", "dv", "dw"), got, ref):
        assert rel(g_, r_) <= FP32_REL, name


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("n,c,h,k", [(2, 12, 4, 4), (1, 20, 12, 8)])
def test_fwd_bwd_bf16_vs_oracle(lcm, algo, n, c, h, k):
    q, kc, vc, idx, w, dout = cases.gca_indexed_case(2, n, c, h, k, dtype=torch.bfloat16)
    ref = G.gca_indexed_grads(q.float(), kc.float(), vc.float(), idx, w, 0.125, dout.float())
    got = run_indexed(lcm, q, kc, vc, idx, w, 0.125, dout=dout, algo=algo)
    for name, g_, r_ in zip(("o", "dq", "dk", "dv", "dw"), got, ref):
        assert rel(g_, r_) <= BF16_REL, name
    assert lcm.read_status() == 0


@pytest.mark.parametrize("name,dtype", [("gca_ref_fp32_gqa4", torch.float32), ("gca_ref_fp32_mha", torch.float32),
                                        ("gca_ref_fp32_gqa2_scale05", torch.float32),
                                        ("gca_ref_bf16_gqa4", torch.bfloat16)])
def test_attention_against_reference_golden(lcm, golden_dir, name, dtype):
    """``attention`` (the 6-argument drop-in) against outputs of the reference's own einsum
    formulation + autograd, including GQA."""
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    seed, z, hq, hkv, k, std, scale = g["meta"]
    q, kk, v, w, dout = cases.gca_gathered_case(int(seed), int(z), int(hq), int(hkv), int(k), std=float(std), dtype=dtype)
    assert abs(cases.checksum(q, kk, v, w, dout) - float(g["in_checksum"])) < 1e-6
    qd, kd, vd, wd = (t.cuda().requires_grad_() for t in (q, kk, v, w))
    out = lcm.attention(qd, kd, vd, wd, float(scale), 0)
    out.backward(dout.cuda())
    tol = FP32_REL if dtype == torch.float32 else BF16_REL
    for name_, got, key in (("o", out, "o"), ("dq", qd.grad, "dq"), ("dk", kd.grad, "dk"), ("dv", vd.grad, "dv"),
                            ("dw", wd.grad, "dw")):
        ref = torch.from_numpy(g[key])
        assert got.shape == ref.shape, name_
        assert rel(got, ref) <= tol, name_
        if dtype == torch.bfloat16:      # the reference test's own absolute tolerances
            atol = 0.5 if key == "dw" else 1e-2
            assert (got.float().cpu() - ref).abs().max().item() <= atol * max(1.0, ref.abs().max().item()), name_


@pytest.mark.parametrize("name,sq", [("gca_ref_inf_q2", 2), ("gca_ref_inf_q1", 1)])
def test_gca_kv_cache_decode_golden(lcm, golden_dir, name, sq):
    """``gca_kv_cache`` with 2 and 1 query rows, GQA 2, sm_scale 0.5 (ltriton/gca.py:963-1011)."""
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    q, kk, v, w, _ = cases.gca_gathered_case(7 + sq, 3, 4, 2, 5, s=sq, std=0.5)
    ref = torch.from_numpy(g["o"])
    out = lcm.gca_kv_cache(q.cuda().bfloat16(), kk.cuda().bfloat16(), v.cuda().bfloat16(), w.cuda(), 0.5, 0.0)
    assert out.shape == ref.shape
    assert (out.float().cpu() - ref).abs().max().item() <= 1e-2
    out32 = lcm.gca_kv_cache(q.cuda(), kk.cuda(), v.cuda(), w.cuda(), 0.5, 0.0)
    assert rel(out32, ref) <= FP32_REL


@pytest.mark.parametrize("sq", [1, 2, 5, 16, 33, 64])
def test_gca_kv_cache_any_query_length(lcm, sq):
    q, kk, v, w, _ = cases.gca_gathered_case(11, 4, 6, 3, 7, s=sq, std=1.0)
    ref = G.gca_gathered(q.bfloat16().float(), kk.bfloat16().float(), v.bfloat16().float(), w, 0.125)
    out = lcm.gca_kv_cache(q.cuda().bfloat16(), kk.cuda().bfloat16(), v.cuda().bfloat16(), w.cuda(), 0.125, 0.0)
    assert rel(out, ref) <= BF16_REL


def test_decode_dynamic_k_and_padding(lcm):
    """While generating, K = min(E, topk) grows 1, 2, 3 ...; unused slots are padding (-1)."""
    g = torch.Generator().manual_seed(5)
    n, c, h = 3, 9, 12
    kc = torch.randn(n, c, 64, h * 64, generator=g).bfloat16()
    vc = torch.randn(n, c, 64, h * 64, generator=g).bfloat16()
    for kvalid in (1, 2, 3, 8):
        q = torch.randn(n, 1, h, 1, 64, generator=g).bfloat16()
        idx = torch.full((n, 1, 8), -1, dtype=torch.int64)
        for b in range(n):
            idx[b, 0, :kvalid] = torch.randperm(c, generator=g)[:kvalid]
        w = torch.zeros(n, 1, 8)
        w[:, :, :kvalid] = torch.softmax(torch.randn(n, 1, kvalid, generator=g), -1)
        ref = G.gca_indexed(q.float(), kc.float(), vc.float(), idx, w, 0.125)
        out = lcm.gca_indexed_nograd(q.cuda(), kc.cuda(), vc.cuda(), idx.cuda(), w.cuda(), 0.125)
        assert rel(out, ref) <= BF16_REL


@pytest.mark.parametrize("hq,hkv,sq,k,obo", [(12, 12, 1, 11, False), (8, 4, 1, 8, False), (8, 4, 2, 5, True), (4, 1, 1, 3, True),
                                            (6, 6, 3, 9, False), (2, 2, 4, 2, False)])
def test_decode_rows_kernel_shapes(lcm, hq, hkv, sq, k, obo):
    """The register-streaming decode kernel (up to four rows per kv head): more slots than warps, padding
    slots, grouped-query heads, two to four rows, the off-by-one softmax, against the oracle."""
    g = torch.Generator().manual_seed(100 * hq + 10 * sq + k)
    n, c = 3, 20
    kc = torch.randn(n, c, 64, hkv * 64, generator=g).bfloat16()
    vc = torch.randn(n, c, 64, hkv * 64, generator=g).bfloat16()
    q = torch.randn(n, 1, hq, sq, 64, generator=g).bfloat16()
    idx = torch.stack([torch.randperm(c, generator=g)[:k] for _ in range(n)]).view(n, 1, k)
    idx[0, 0, k - 1] = -1                                    # a padding slot
    w = torch.softmax(torch.randn(n, 1, k, generator=g), -1)
    ref = G.gca_indexed(q.float(), kc.float(), vc.float(), idx, w, 0.125, off_by_one=1.0 if obo else 0.0)
    out = lcm.gca_indexed_nograd(q.cuda(), kc.cuda(), vc.cuda(), idx.cuda(), w.cuda(), 0.125, softmax_off_by_one=obo)
    assert out.shape == ref.shape
    assert rel(out, ref) <= BF16_REL
    assert lcm.read_status() == 0


@pytest.mark.parametrize("algo", ALGOS)
def test_indexed_equals_gathered_and_scatter_add(lcm, algo):
    """gca_indexed(cache, idx) == attention(gather(cache, idx)); dK/dV into the cache equal
    the index_put_(accumulate=True) scatter of the gathered gradients (DRT.py:193-199)."""
    n, c, h, k = 2, 10, 4, 4
    q, kc, vc, idx, w, dout = cases.gca_indexed_case(3, n, c, h, k, dtype=torch.bfloat16)
    # force duplicates: many query chunks retrieve chunk 0
    idx[:, 2:, 0] = 0
    idx[:, 3:, 1] = 1
    o, dq, dk, dv, dw = run_indexed(lcm, q, kc, vc, idx, w, 0.125, dout=dout, algo=algo)
    ref = G.gca_indexed_grads(q.float(), kc.float(), vc.float(), idx, w, 0.125, dout.float())
    for name, g_, r_ in zip(("o", "dq", "dk", "dv", "dw"), (o, dq, dk, dv, dw), ref):
        assert rel(g_, r_) <= BF16_REL, name
    # the gathered route through the 6-argument drop-in
    gk, gv = G.gather_chunks(kc, vc, idx, h)
    wz = torch.where(idx < 0, torch.zeros_like(w), w).reshape(-1, k)
    o2 = lcm.attention(q.reshape(-1, h, 64, 64).cuda(), gk.cuda(), gv.cuda(), wz.cuda(), 0.125, 0.0)
    assert rel(o2.reshape(o.shape), o) <= 1e-2


@pytest.mark.parametrize("algo", ALGOS)
def test_true_off_by_one_and_inert_sm_n(lcm, algo):
    q, kc, vc, idx, w, dout = cases.gca_indexed_case(4, 2, 8, 2, 4, dtype=torch.bfloat16, zero_landmark=False)
    # sm_n alone changes nothing (reference kernels: ltriton/gca.py:48-49,187)
    a = run_indexed(lcm, q, kc, vc, idx, w, 0.125, algo=algo)
    b = lcm.gca_indexed(q.cuda(), kc.cuda(), vc.cuda(), idx.cuda(), w.cuda(), 0.125, 1.0, algo=algo)
    assert torch.equal(a, b)
    ref = G.gca_indexed_grads(q.float(), kc.float(), vc.float(), idx, w, 0.125, dout.float(), off_by_one=1.0)
    got = run_indexed(lcm, q, kc, vc, idx, w, 0.125, dout=dout, algo=algo, softmax_off_by_one=True)
    for name, g_, r_ in zip(("o", "dq", "dk", "dv", "dw"), got, ref):
        assert rel(g_, r_) <= BF16_REL, name


@pytest.mark.parametrize("algo", ALGOS)
def test_lse_and_padding_slots(lcm, algo):
    from long_context_modeling_b200 import gca as gmod
    q, kc, vc, idx, w, _ = cases.gca_indexed_case(6, 1, 6, 2, 4, dtype=torch.bfloat16)
    out, lse = gmod.gca_forward_with_lse(q.cuda(), kc.cuda(), vc.cuda(), idx.cuda(), w.cuda(), 0.125, algo=algo)
    gk, _ = G.gather_chunks(kc.float(), vc.float(), idx, 2)
    ref = G.gca_lse(q.float().reshape(-1, 2, 64, 64), gk, 0.125)          # (Z, Hq, K, S)
    pad = (idx < 0).reshape(-1, 1, 4, 1).expand_as(ref)
    assert torch.all(lse.cpu()[pad] == 0)
    assert (lse.cpu()[~pad] - ref[~pad]).abs().max().item() <= 2e-2


@pytest.mark.parametrize("algo", ALGOS)
def test_out_of_range_index_is_flagged_not_read(lcm, algo):
    q, kc, vc, idx, w, _ = cases.gca_indexed_case(7, 1, 6, 2, 4, dtype=torch.bfloat16)
    good = run_indexed(lcm, q, kc, vc, idx, w, 0.125, algo=algo)
    assert lcm.read_status() == 0
    bad = idx.clone()
    bad[0, 4, 1] = 1000                 # >= C: skipped and reported
    w2 = w.clone()
    out = run_indexed(lcm, q, kc, vc, bad, w2, 0.125, algo=algo)
    assert lcm.read_status() & 1
    assert torch.equal(out[0, :4], good[0, :4])


@pytest.mark.parametrize("algo", ALGOS)
def test_determinism(lcm, algo):
    q, kc, vc, idx, w, dout = cases.gca_indexed_case(8, 2, 16, 4, 8, dtype=torch.bfloat16)
    a = run_indexed(lcm, q, kc, vc, idx, w, 0.125, dout=dout, algo=algo)
    b = run_indexed(lcm, q, kc, vc, idx, w, 0.125, dout=dout, algo=algo)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


@pytest.mark.parametrize("algo", ALGOS)
def test_backward_stage_by_stage_equals_one_call(lcm, algo):
    """gca_bwd_stages: index, then the dQ/dw stage, then the dK/dV stage give the bits of the
    single gca_bwd call."""
    from long_context_modeling_b200 import gca as gmod
    q, kc, vc, idx, w, dout = (t.cuda() for t in cases.gca_indexed_case(21, 2, 14, 4, 8, dtype=torch.bfloat16))
    _, lse = gmod.gca_forward_with_lse(q, kc, vc, idx, w, 0.125, algo=algo)
    full = gmod.gca_backward_stages(q, kc, vc, idx, w, dout, lse, 0.125, algo=algo)
    bufs = gmod.gca_backward_stages(q, kc, vc, idx, w, dout, lse, 0.125, stages=gmod.BWD_STAGE_INDEX, algo=algo)
    for t in bufs[:4]:
        t.fill_(7)                                       # stale contents must be overwritten
    gmod.gca_backward_stages(q, kc, vc, idx, w, dout, lse, 0.125, stages=gmod.BWD_STAGE_Q, bufs=bufs, algo=algo)
    gmod.gca_backward_stages(q, kc, vc, idx, w, dout, lse, 0.125, stages=gmod.BWD_STAGE_KV, bufs=bufs, algo=algo)
    torch.cuda.synchronize()
    for x, y in zip(full, bufs[:4]):
        assert torch.equal(x, y)
    assert lcm.read_status() == 0


@pytest.mark.parametrize("shape", [(2, 14, 4, 8), (3, 40, 2, 4), (1, 70, 4, 16), (8, 256, 2, 8), (1, 1024, 2, 4)])
def test_inverse_index_single_launch_equals_radix_sort(lcm, shape):
    """The single-launch counting sort that builds the inverse retrieval index for small problems
    (stable by (query chunk, slot) inside a chunk; units walked by decreasing number of
    retrievers) gives the bits of the radix-sort path: same entry order means the same float32
    accumulation order in dK / dV."""
    from long_context_modeling_b200 import gca as gmod
    n, c, h, k = shape
    q, kc, vc, idx, w, dout = (t.cuda() for t in cases.gca_indexed_case(41, n, c, h, k, dtype=torch.bfloat16))
    idx = idx.clone()
    idx[:, c // 2:, 0] = 0                               # many retrievers of one chunk
    idx[:, -1, 1:] = -1                                  # padding slots
    _, lse = gmod.gca_forward_with_lse(q, kc, vc, idx, w, 0.125)
    fast = gmod.gca_backward_stages(q, kc, vc, idx, w, dout, lse, 0.125)
    slow = gmod.gca_backward_stages(q, kc, vc, idx, w, dout, lse, 0.125, stages=gmod.BWD_STAGE_ALL | gmod.BWD_INDEX_BY_SORT)
    torch.cuda.synchronize()
    for x, y in zip(fast, slow):
        assert torch.equal(x, y)
    assert lcm.read_status() == 0


def test_host_pipeline_matches_direct_calls(lcm):
    """HostGcaPipeline (upload / kernels / download of consecutive steps overlapped on three
    streams) returns, step by step and in order, the bits of the plain calls."""
    steps = [cases.gca_indexed_case(30 + i, 2, 10, 4, 4, dtype=torch.bfloat16) for i in range(5)]
    host = [tuple(t.pin_memory() for t in (q, kc, vc, idx.to(torch.int32), w, dout)) for q, kc, vc, idx, w, dout in steps]
    want = [run_indexed(lcm, q, kc, vc, idx, w, 0.125, dout=dout) for q, kc, vc, idx, w, dout in steps]
    pipe = lcm.HostGcaPipeline(torch.device("cuda", 0), 0.125, depth=2)
    got = []
    for hs in host:
        done = pipe.submit(hs)
        if done is not None:
            got.append([t.clone() for t in done])
    got += [[t.clone() for t in done] for done in pipe.drain()]
    assert len(got) == len(want)
    for g_, w_ in zip(got, want):
        for x, y in zip(g_, w_):
            assert torch.equal(x, y.cpu())
    assert pipe.h2d_bytes > 0 and pipe.d2h_bytes > 0


def test_strided_query_view_and_token_major_output(lcm):
    """q as a strided view of a (N, C, S, H*D) projection output, skipping chunk 0, and the
    output written token-major: no layout copies on either side."""
    n, c, h, k = 2, 7, 4, 3
    g = torch.Generator().manual_seed(12)
    proj = torch.randn(n, c, 64, h * 64, generator=g).bfloat16()
    _, kc, vc, idx, w, _ = cases.gca_indexed_case(12, n, c, h, k, dtype=torch.bfloat16)
    q5 = proj.view(n, c, 64, h, 64).permute(0, 1, 3, 2, 4)[:, 1:]
    ref = G.gca_indexed(q5.float(), kc.float(), vc.float(), idx, w, 0.125)
    out = lcm.gca_indexed(q5.cuda(), kc.cuda(), vc.cuda(), idx.cuda(), w.cuda(), 0.125, token_major_out=True)
    assert out.permute(0, 1, 3, 2, 4).is_contiguous()
    assert rel(out, ref) <= BF16_REL


def test_single_head_units_match_head_pairs(lcm):
    """The tensor-core forward with one head per work unit (GCA_ALGO_TC_UNPAIRED) gives the same
    bits as the paired layout: both run the same per-row arithmetic."""
    q, kc, vc, idx, w, _ = cases.gca_indexed_case(9, 1, 8, 3, 4, dtype=torch.bfloat16)
    a = run_indexed(lcm, q, kc, vc, idx, w, 0.125, algo=2)
    b = run_indexed(lcm, q, kc, vc, idx, w, 0.125, algo=3)          # GCA_ALGO_TC_UNPAIRED
    assert torch.equal(a, b)


def test_module_drop_in_matches_indexed_path(lcm):
    """TritonGroupCrossAttention.forward (pre-gathered, reference argument meaning) and
    forward_indexed (cache + indices) agree, in train and eval mode."""
    torch.manual_seed(0)
    n, c, h, k, dim = 2, 6, 2, 3, 128
    mod = lcm.TritonGroupCrossAttention(dim, h, 63, k).cuda().bfloat16()
    g = torch.Generator().manual_seed(13)
    hidden = torch.randn(n, c, 64, dim, generator=g).bfloat16().cuda()
    kc = torch.randn(n, c, 64, dim, generator=g).bfloat16().cuda()
    vc = torch.randn(n, c, 64, dim, generator=g).bfloat16().cuda()
    idx, scores = cases.causal_indices(g, n, c, k)
    w = torch.nan_to_num(torch.softmax(scores, -1), nan=0.0).cuda()
    gk, gv = G.gather_chunks(kc, vc, idx.cuda(), h)
    wz = w.reshape(-1, k)
    for train in (True, False):
        mod.train(train)
        a = mod(hidden, gk, gv, wz)
        b = mod.forward_indexed(hidden, kc, vc, idx.cuda(), w)
        assert a.shape == (n, c * 64, dim)
        assert a[:, :64].abs().max().item() == 0
        assert rel(a, b) <= 2e-2


def test_flash_layout_module_matches_triton_layout_module(lcm):
    """GroupCrossAttention (the reference's flash-attn variant: chunks as (N*D*K, S, h, d), weights
    (N, D, K), model/DRT.py:235-302) gives the bits of TritonGroupCrossAttention on the same
    parameters and data, forward and backward."""
    torch.manual_seed(1)
    n, c, h, k, dim = 2, 5, 2, 4, 128
    a_mod = lcm.TritonGroupCrossAttention(dim, h, 63, k).cuda().bfloat16()
    b_mod = lcm.GroupCrossAttention(dim, h, 63, k).cuda().bfloat16()
    b_mod.load_state_dict(a_mod.state_dict())
    g = torch.Generator().manual_seed(17)
    hidden = torch.randn(n, c, 64, dim, generator=g).bfloat16().cuda()
    kc = torch.randn(n, c, 64, dim, generator=g).bfloat16().cuda()
    vc = torch.randn(n, c, 64, dim, generator=g).bfloat16().cuda()
    idx, scores = cases.causal_indices(g, n, c, k)
    w = torch.nan_to_num(torch.softmax(scores, -1), nan=0.0).cuda()
    safe = idx.clamp(min=0).cuda()                                    # padding slots carry weight 0
    gathered_k = torch.stack([kc[b][safe[b].reshape(-1)] for b in range(n)])      # (N, D'*K, S, dim)
    gathered_v = torch.stack([vc[b][safe[b].reshape(-1)] for b in range(n)])
    tk, tv, tw = a_mod.preprocess_chunk_kv_cache(gathered_k, gathered_v, w, h)
    fk, fv, fw = b_mod.preprocess_chunk_kv_cache(gathered_k, gathered_v, w, h)
    assert fk.shape == (n * (c - 1) * k, 64, h, dim // h) and fw.shape == w.shape
    outs = []
    for mod, args in ((a_mod, (tk, tv, tw)), (b_mod, (fk, fv, fw))):
        mod.zero_grad()
        hs = hidden.clone().requires_grad_()
        o = mod(hs, *args)
        o.float().square().sum().backward()
        outs.append((o, hs.grad, mod.q_proj.weight.grad.clone()))
    for x, y in zip(*outs):
        assert torch.equal(x, y)
    assert outs[0][0].shape == (n, c * 64, dim)


def test_full_size_config_properties(lcm):
    """BASELINE sweep point 16K tokens, B*H = 96, K = 8 (too large for the CPU oracle as a
    whole): size-independent properties + a sample of units against the oracle."""
    n, c, h, k = 8, 256, 12, 8
    g = torch.Generator().manual_seed(0)
    dev = "cuda"
    q = torch.randn(n, c - 1, h, 64, 64, generator=g).bfloat16().to(dev)
    kc = torch.randn(n, c, 64, h * 64, generator=g).bfloat16().to(dev)
    vc = torch.randn(n, c, 64, h * 64, generator=g).bfloat16().to(dev)
    idx, scores = cases.causal_indices(g, n, c, k)
    w = torch.nan_to_num(torch.softmax(scores, -1), nan=0.0)
    idx_d, w_d = idx.to(dev), w.to(dev)
    out = lcm.gca_indexed_nograd(q, kc, vc, idx_d, w_d, 0.125)
    # (1) sampled units against the oracle
    for (b, j) in ((0, 0), (0, 1), (3, 100), (7, 254), (5, 9)):
        ref = G.gca_indexed(q[b:b + 1, j:j + 1].float().cpu(), kc[b:b + 1].float().cpu(), vc[b:b + 1].float().cpu(),
                            idx[b:b + 1, j:j + 1], w[b:b + 1, j:j + 1], 0.125)
        assert rel(out[b:b + 1, j:j + 1], ref) <= BF16_REL or ref.abs().max() == 0
    # (2) linearity in the retrieval weights: out(w1) + out(w2) == out(w1 + w2) within rounding
    w1 = w_d * 0.25
    w2 = w_d * 0.75
    o12 = lcm.gca_indexed_nograd(q, kc, vc, idx_d, w1, 0.125).float() + lcm.gca_indexed_nograd(q, kc, vc, idx_d, w2, 0.125).float()
    assert rel(o12, out) <= 2e-2
    # (3) zero weights -> exact zeros; one-hot weight -> plain attention over that chunk
    assert lcm.gca_indexed_nograd(q, kc, vc, idx_d, torch.zeros_like(w_d), 0.125).abs().max().item() == 0
    # (4) permuting the K slots of every row does not change the result beyond rounding
    perm = torch.randperm(k, generator=g)
    o_perm = lcm.gca_indexed_nograd(q, kc, vc, idx_d[..., perm].contiguous(), w_d[..., perm].contiguous(), 0.125)
    assert rel(o_perm, out) <= 1e-2
    # (5) backward at full size: sum of dw over slots equals <dout, out> summed per row block
    qg = q.clone().requires_grad_()
    kg = kc.clone().requires_grad_()
    vg = vc.clone().requires_grad_()
    wg = w_d.clone().requires_grad_()
    o = lcm.gca_indexed(qg, kg, vg, idx_d, wg, 0.125)
    dout = torch.randn(o.shape, generator=g).bfloat16().to(dev)
    o.backward(dout)
    lhs = (wg.grad * w_d).sum(-1)                                   # sum_k w_k <dO, O_k> = <dO, O>
    rhs = (dout.float() * o.float()).sum(dim=(2, 3, 4))
    assert ((lhs - rhs).abs().max() / (rhs.abs().max() + 1e-6)).item() <= 3e-2
    # never-retrieved chunks get exactly zero gradient
    used = torch.zeros(n, c, dtype=torch.bool)
    for b in range(n):
        used[b, idx[b][idx[b] >= 0]] = True
    assert kg.grad.view(n, c, -1)[~used.to(dev)].abs().max().item() == 0
    assert lcm.read_status() == 0
