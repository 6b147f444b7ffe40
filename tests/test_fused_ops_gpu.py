"""The projections either side of GCA with their small operations fused in (inference path):
``gca_row_rms`` + ``gca_linear`` through the C ABI, against plain float32 PyTorch on the same bf16
inputs, and ``TritonGroupCrossAttention.forward_fused`` against the fixture produced by the
REFERENCE's module class (``tests/golden/module_ref.npz``, ``model/DRT.py:345-398``) and against
this repository's unfused ``forward_indexed``.  bf16 data, float32 accumulation: per element
|a - b| <= 1e-2 * scale + 2e-2 * |b| with scale = max |b|.
"""
import os

import numpy as np
import pytest
import torch

import make_golden as MG

pytestmark = pytest.mark.gpu


def close(a, b, what=""):
    a, b = a.detach().float().cpu(), torch.as_tensor(b).float().cpu()
    scale = b.abs().max().item() + 1e-12
    bad = (a - b).abs() > 1e-2 * scale + 2e-2 * b.abs()
    assert not bad.any(), (what, int(bad.sum()), ((a - b).abs().max() / scale).item())


def need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


@pytest.mark.parametrize("m,d", [(1, 768), (37, 128), (4100, 768)])
def test_row_rms(m, d):
    need_gpu()
    from long_context_modeling_b200 import fused_ops as F
    x = (torch.randn(m, d, generator=torch.Generator().manual_seed(m)) * 3).bfloat16().cuda()
    got = F.row_rms(x, 1e-5)
    ref = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
    assert torch.allclose(got, ref, rtol=1e-5, atol=0)


@pytest.mark.parametrize("m,n,k", [(1, 768, 768), (300, 768, 768), (129, 48, 128), (1000, 1024, 3072), (64, 272, 64)])
@pytest.mark.parametrize("with_scale,with_res", [(False, False), (True, False), (False, True), (True, True)])
def test_linear_against_float32(m, n, k, with_scale, with_res):
    need_gpu()
    from long_context_modeling_b200 import fused_ops as F
    import long_context_modeling_b200 as lcm
    g = torch.Generator().manual_seed(m * 7 + n)
    x = torch.randn(m, k, generator=g).bfloat16().cuda()
    w = (torch.randn(n, k, generator=g) / k ** 0.5).bfloat16().cuda()
    sc = (torch.rand(m, generator=g) + 0.5).cuda() if with_scale else None
    res = torch.randn(m, n, generator=g).bfloat16().cuda() if with_res else None
    out = torch.full((m, n), 7.0, dtype=torch.bfloat16, device="cuda")
    F.linear(x, w, row_scale=sc, residual=res, out=out)
    ref = x.float() @ w.float().T
    if with_scale:
        ref = ref * sc[:, None]
    if with_res:
        ref = ref + res.float()
    close(out, ref, (m, n, k))
    assert lcm.read_status() == 0


def test_linear_writes_only_its_rows_and_columns():
    """Strided output (a column block of a wider matrix, a row block of a taller one): nothing outside
    the (M, N) window changes."""
    need_gpu()
    from long_context_modeling_b200 import fused_ops as F
    g = torch.Generator().manual_seed(3)
    x = torch.randn(200, 128, generator=g).bfloat16().cuda()
    w = (torch.randn(64, 128, generator=g) / 11).bfloat16().cuda()
    big = torch.full((260, 256), -5.0, dtype=torch.bfloat16, device="cuda")
    F.linear(x, w, out=big[30:230, 64:128])
    close(big[30:230, 64:128], x.float() @ w.float().T)
    mask = torch.ones_like(big, dtype=torch.bool)
    mask[30:230, 64:128] = False
    assert (big[mask] == -5.0).all()


def test_linear_rejects_bad_arguments():
    need_gpu()
    from long_context_modeling_b200 import fused_ops as F
    x = torch.zeros(8, 96, dtype=torch.bfloat16, device="cuda")            # K not a multiple of 64
    w = torch.zeros(64, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        F.linear(x, w)
    with pytest.raises(ValueError):
        F.linear(torch.zeros(8, 128, device="cuda"), torch.zeros(64, 128, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(RuntimeError):
        F.linear(torch.zeros(8, 128, dtype=torch.bfloat16), torch.zeros(64, 128, dtype=torch.bfloat16))


def test_rmsnorm_linear_matches_norm_then_projection():
    need_gpu()
    from long_context_modeling_b200 import fused_ops as F
    g = torch.Generator().manual_seed(9)
    x = (torch.randn(2, 5, 64, 768, generator=g) * 2).bfloat16().cuda()
    gain = (1 + 0.2 * torch.randn(768, generator=g)).cuda()
    w = (torch.randn(768, 768, generator=g) / 28).bfloat16().cuda()
    got = F.rmsnorm_linear(x, F.fold_gain(w, gain), 1e-5)
    xf = x.float()
    normed = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * gain
    close(got, normed @ w.float().T)
    assert got.shape == (2, 5, 64, 768)


def _fixture_module(golden_dir):
    import long_context_modeling_b200 as lcm
    g = np.load(os.path.join(golden_dir, "module_ref.npz"))
    cfg = MG.ModuleConfig()
    n, c, k = 1, 3, cfg.chunk_topk
    hidden, gk, gv, w, dout, params = MG.module_case(51, n, c, cfg.num_attention_heads, k, cfg.hidden_size)
    mod = lcm.TritonGroupCrossAttention(cfg).cuda()
    mod.load_state_dict({k_: v_.cuda() for k_, v_ in params.items()})
    return g, cfg, mod.bfloat16().eval(), hidden, gk, gv, w


def test_fused_module_path_matches_reference_class(golden_dir):
    """forward_fused (RMSNorm folded into q_proj's GEMM, o_proj with residual epilogue) in bf16 against
    the reference class's float32 output for the same parameters and inputs; the gathered chunks of
    the fixture serve as the cache, read through an identity index."""
    need_gpu()
    g, cfg, mod, hidden, gk, gv, w = _fixture_module(golden_dir)
    k = cfg.chunk_topk
    n, dk = gk.shape[:2]
    idx = torch.arange(dk, dtype=torch.int32).view(1, dk // k, k).expand(n, -1, -1).contiguous().cuda()
    hs = hidden.bfloat16().cuda()
    kc, vc = gk.bfloat16().cuda(), gv.bfloat16().cuda()
    with torch.no_grad():
        o = mod.forward_fused(hs, kc, vc, idx, w.cuda())
        close(o, g["triton_eval_o"], "no residual")
        assert o[:, :64].abs().max().item() == 0            # the first chunk retrieves nothing
        res = torch.randn(o.shape, generator=torch.Generator().manual_seed(1)).bfloat16().cuda()
        o2 = mod.forward_fused(hs, kc, vc, idx, w.cuda(), residual=res)
        close(o2, torch.as_tensor(g["triton_eval_o"]) + res.float().cpu(), "with residual")
        assert torch.equal(o2[:, :64], res[:, :64])
        # and against the unfused path of this repository
        close(o2, (mod.forward_indexed(hs, kc, vc, idx, w.cuda()).float() + res.float()), "vs forward_indexed")
        # one-row decode step (chunk_size == 1: nothing is skipped)
        o1 = mod.forward_fused(hs[:, 1:2, :1], kc[:, :k], vc[:, :k], idx[:, :1], w[:, :1].cuda())
        close(o1, g["triton_decode_o"], "decode")


def _window_reference(q, k, v, window, slopes, scale):
    """float32: explicit scores, ALiBi bias, window + causal mask, softmax (model/llama.py:684-688 semantics)."""
    n, hq, sq, d = q.shape
    hkv, t = k.shape[1], k.shape[2]
    g = hq // hkv
    kf = k.float().repeat_interleave(g, 1)
    vf = v.float().repeat_interleave(g, 1)
    s = torch.einsum("nhid,nhjd->nhij", q.float(), kf) * scale
    pos = torch.arange(t - sq, t).view(sq, 1)
    j = torch.arange(t).view(1, t)
    dist = (pos - j).float()
    bias = torch.zeros(hq, sq, t) if slopes is None else -slopes.view(hq, 1, 1).cpu() * dist
    bias = bias.masked_fill((dist < 0) | (dist > window), float("-inf"))
    p = torch.softmax(s.cpu() + bias, -1)
    return torch.einsum("nhij,nhjd->nhid", p, vf.cpu())


@pytest.mark.parametrize("n,hq,hkv,sq,t,window,alibi", [
    (2, 12, 12, 1, 513, 512, True),       # the model's decode step: one new position, full window
    (3, 4, 4, 2, 300, 512, True),         # two new positions, fewer keys than the window
    (2, 8, 4, 2, 700, 128, True),         # grouped-query heads, keys older than the window are skipped
    (1, 2, 2, 1, 1, 16, False),           # a single key, no ALiBi
    (2, 4, 1, 1, 97, 40, True),           # four q heads on one kv head
    (1, 12, 12, 3, 1030, 512, True),      # three rows
])
def test_window_decode_against_float32(n, hq, hkv, sq, t, window, alibi):
    need_gpu()
    from long_context_modeling_b200 import fused_ops as F
    g = torch.Generator().manual_seed(t + sq)
    q = torch.randn(n, hq, sq, 64, generator=g).bfloat16().cuda()
    k = torch.randn(n, hkv, t, 64, generator=g).bfloat16().cuda()
    v = torch.randn(n, hkv, t, 64, generator=g).bfloat16().cuda()
    slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / hq) for i in range(hq)]).cuda() if alibi else None
    got = F.window_decode(q, k, v, window, slopes, 0.125)
    ref = _window_reference(q, k, v, window, slopes, 0.125)
    close(got, ref, (n, hq, hkv, sq, t, window))


def test_window_decode_reads_strided_caches():
    """k / v as (N, T, H, 64) token-major storage viewed as (N, H, T, 64): the reference's cache layout."""
    need_gpu()
    from long_context_modeling_b200 import fused_ops as F
    g = torch.Generator().manual_seed(5)
    q = torch.randn(2, 1, 6, 64, generator=g).bfloat16().cuda().transpose(1, 2)          # (N, H, 1, 64) view
    k = torch.randn(2, 200, 6, 64, generator=g).bfloat16().cuda().transpose(1, 2)
    v = torch.randn(2, 200, 6, 64, generator=g).bfloat16().cuda().transpose(1, 2)
    slopes = torch.full((6,), 0.05).cuda()
    close(F.window_decode(q, k, v, 64, slopes, 0.125), _window_reference(q, k, v, 64, slopes, 0.125))


@pytest.mark.parametrize("m,v,k", [(300, 50265, 768), (1, 1000, 64), (129, 257, 128), (2000, 4096, 768)])
def test_linear_cross_entropy_against_float32(m, v, k):
    """LM head + cross-entropy without logits in memory, against torch on float32 logits of the same
    bf16 inputs; ignored rows (target -100) give 0."""
    need_gpu()
    from long_context_modeling_b200 import fused_ops as F
    import long_context_modeling_b200 as lcm
    g = torch.Generator().manual_seed(m + v)
    x = torch.randn(m, k, generator=g).bfloat16().cuda()
    w = (torch.randn(v, k, generator=g) * (3.0 / k ** 0.5)).bfloat16().cuda()
    t = torch.randint(0, v, (m,), generator=g).cuda()
    if m > 4:
        t[3] = -100
        t[m - 1] = v - 1
    loss, lse = F.linear_cross_entropy(x, w, t, return_lse=True)
    logits = x.float() @ w.float().T
    ref = torch.nn.functional.cross_entropy(logits, t, reduction="none", ignore_index=-100)
    assert torch.allclose(loss, ref, rtol=2e-4, atol=2e-4), (loss - ref).abs().max().item()
    assert torch.allclose(lse, torch.logsumexp(logits, -1), rtol=2e-5, atol=2e-4)
    if m > 4:
        assert loss[3].item() == 0.0
    assert lcm.read_status() == 0


def test_linear_cross_entropy_with_rmsnorm_scale_and_bad_target():
    need_gpu()
    from long_context_modeling_b200 import fused_ops as F
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(2, 70, 128, generator=g) * 2).bfloat16().cuda()
    w = (torch.randn(513, 128, generator=g) / 4).bfloat16().cuda()
    t = torch.randint(0, 513, (2, 70), generator=g).cuda()
    sc = F.row_rms(x, 1e-5)
    loss = F.linear_cross_entropy(x, w, t, row_scale=sc)
    xf = x.float()
    logits = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)) @ w.float().T
    ref = torch.nn.functional.cross_entropy(logits.view(-1, 513), t.view(-1), reduction="none").view(2, 70)
    assert loss.shape == (2, 70)
    assert torch.allclose(loss, ref, rtol=3e-4, atol=3e-4)
    t[0, 0] = 513                                   # outside the vocabulary: the loss says so
    assert torch.isnan(F.linear_cross_entropy(x, w, t)[0, 0])


@pytest.mark.parametrize("n,h,t", [(2, 3, 513), (1, 1, 1), (3, 2, 41), (2, 12, 640)])
def test_window_shift_append_in_place(n, h, t):
    """Oldest row out, new row in, in place, against torch.cat + slice; batch-strided windows and new rows that
    are views of a wider projection output."""
    need_gpu()
    from long_context_modeling_b200 import fused_ops as F
    g = torch.Generator().manual_seed(t)
    big_k = torch.randn(n + 1, h, t, 64, generator=g).bfloat16().cuda()
    big_v = torch.randn(n + 1, h, t, 64, generator=g).bfloat16().cuda()
    kw, vw = big_k[1:], big_v[1:]                                   # views with an offset
    qkv = torch.randn(n, 3 * h * 64, generator=g).bfloat16().cuda()
    kn = qkv[:, h * 64:2 * h * 64].view(n, 1, h, 64).transpose(1, 2)  # (N, H, 1, 64) strided views
    vn = qkv[:, 2 * h * 64:].view(n, 1, h, 64).transpose(1, 2)
    ref_k, ref_v = torch.cat([kw, kn], 2)[:, :, 1:].clone(), torch.cat([vw, vn], 2)[:, :, 1:].clone()
    guard = big_k[0].clone()
    F.window_shift_append(kw, vw, kn, vn)
    assert torch.equal(kw, ref_k) and torch.equal(vw, ref_v)
    assert torch.equal(big_k[0], guard)                              # nothing outside the windows moved


@pytest.mark.gpu
@pytest.mark.parametrize("n,hq,hkv,t,steps", [(3, 2, 2, 41, 5), (2, 4, 2, 64, 70), (32, 12, 12, 513, 3)])
def test_window_ring_decode_equals_shift_then_decode(n, hq, hkv, t, steps):
    """The ring form (new row replaces the oldest inside the attention kernel, a device counter gives the
    phase) against moving the window and attending to it, step by step: outputs equal within bf16 rounding
    (the keys reach the online softmax in another order), and the ring rolled back by the phase IS the moved
    window -- also after the counter has wrapped around the ring."""
    need_gpu()
    from long_context_modeling_b200 import fused_ops as F
    g = torch.Generator().manual_seed(t + steps)
    ring_k = torch.randn(n, hkv, t, 64, generator=g).bfloat16().cuda()
    ring_v = torch.randn(n, hkv, t, 64, generator=g).bfloat16().cuda()
    lin_k, lin_v = ring_k.clone(), ring_v.clone()
    slopes = (2.0 ** -torch.arange(1, hq + 1).float()).cuda()
    written = torch.zeros(1, dtype=torch.int64, device="cuda")
    for s in range(steps):
        qkv = torch.randn(n, (hq + 2 * hkv) * 64, generator=g).bfloat16().cuda()
        q = qkv[:, :hq * 64].view(n, 1, hq, 64).transpose(1, 2)
        kn = qkv[:, hq * 64:(hq + hkv) * 64].view(n, 1, hkv, 64).transpose(1, 2)
        vn = qkv[:, (hq + hkv) * 64:].view(n, 1, hkv, 64).transpose(1, 2)
        F.window_shift_append(lin_k, lin_v, kn, vn)
        want = F.window_decode(q, lin_k, lin_v, t - 1, slopes, 0.125)
        got = F.window_ring_decode(q, ring_k, ring_v, kn, vn, written, t - 1, slopes, 0.125)
        written += 1
        assert (got.float() - want.float()).abs().max().item() <= 1e-2 * want.float().abs().max().item(), s
    assert torch.equal(torch.roll(ring_k, -(steps % t), 2), lin_k)
    assert torch.equal(torch.roll(ring_v, -(steps % t), 2), lin_v)


@pytest.mark.gpu
def test_window_ring_decode_rejects_bad_arguments():
    need_gpu()
    from long_context_modeling_b200 import fused_ops as F
    q = torch.zeros(1, 1, 1, 64, dtype=torch.bfloat16, device="cuda")
    ring = torch.zeros(1, 1, 8, 64, dtype=torch.bfloat16, device="cuda")
    new = torch.zeros(1, 1, 64, dtype=torch.bfloat16, device="cuda")
    cnt = torch.zeros(1, dtype=torch.int64, device="cuda")
    with pytest.raises(ValueError):
        F.window_ring_decode(q, ring, ring, new, new, cnt.int(), 7)                    # counter must be int64
    with pytest.raises(ValueError):
        F.window_ring_decode(q, ring, ring, new, new, cnt, 3)                          # rows of the ring outside the window
    with pytest.raises(ValueError):
        F.window_ring_decode(q.expand(1, 1, 2, 64).contiguous(), ring, ring, new, new, cnt, 7)      # one new position only


@pytest.mark.gpu
@pytest.mark.parametrize("m,inter", [(1, 8), (32, 2048), (257, 1536)])
def test_silu_mul_against_float32(m, inter):
    """silu(gate) * up over the output of one stacked gate|up projection, against float32 (one bf16 rounding),
    from a row-strided input; argument checks."""
    need_gpu()
    from long_context_modeling_b200 import fused_ops as F
    g = torch.Generator().manual_seed(m + inter)
    wide = (torch.randn(m, 2 * inter + 16, generator=g) * 3).bfloat16().cuda()
    gu = wide[:, :2 * inter]                                        # row stride wider than the row
    want = torch.nn.functional.silu(gu[:, :inter].float()) * gu[:, inter:].float()
    got = F.silu_mul(gu)
    assert got.shape == (m, inter) and got.dtype == torch.bfloat16
    assert (got.float() - want).abs().max().item() <= 1e-2 * want.abs().max().item()
    assert torch.equal(F.silu_mul(gu.view(1, m, 2 * inter).contiguous()).view(m, inter), got)
    with pytest.raises(ValueError):
        F.silu_mul(gu[:, :2 * inter - 8].contiguous()[:, :2 * inter - 12])   # halves not a multiple of 8 wide
