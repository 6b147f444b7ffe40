"""GCA parity with MANY units per persistent CTA.

The tensor-core kernels are persistent: at most one CTA per SM walks a list of units and carries
ring phases, accumulator hand-backs and double buffers from one unit to the next.  These tests
compare out, dq, dk, dv and dw with the CPU oracle (the reference's einsum formulation,
``ltriton/gca.py:912-926``) on problems with several hundred to several thousand units, so that
every CTA processes many units in a row, and on the slot counts, head groupings and head counts
the small cases leave out.

Two criteria per tensor:
* ``rel``: max|a-b| / max|b|  <= 2e-2 (bf16) or 1e-4 (fp32);
* per element: |a-b| <= atol + 2e-2 |b| with atol = 1e-2 * max(1, rms(b)): the reference test's
  own ``atol=1e-2`` (``ltriton/gca.py:938-961``) holds for its N(0, 0.5) inputs, whose outputs have
  rms <= 1; gradients of N(0, 1) inputs summed over many retrievers have rms of 5-30 and are
  rounded to bf16 (2^-9 relative), hence the scaling by the tensor's own rms.
"""
import pytest
import torch

import cases
from oracle import gca_oracle as G

pytestmark = pytest.mark.gpu

NAMES = ("o", "dq", "dk", "dv", "dw")


@pytest.fixture(scope="module")
def lcm():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import long_context_modeling_b200 as m
    return m


def check(name, got, ref, rel_tol, rtol=2e-2, atol=1e-2):
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got.shape == ref.shape, name
    assert torch.isfinite(got).all(), name
    err = (got - ref).abs()
    rel = (err.max() / (ref.abs().max() + 1e-12)).item()
    assert rel <= rel_tol, (name, "rel", rel)
    rms = ref.square().mean().sqrt().item()
    bound = atol * max(1.0, rms) + rtol * ref.abs()
    worst = (err - bound).max().item()
    assert worst <= 0, (name, "per-element excess", worst, "rms", rms)


def run(lcm, q, kc, vc, idx, w, dout, scale=0.125, **kw):
    qd, kd, vd, wd = (t.cuda().requires_grad_() for t in (q, kc, vc, w))
    o = lcm.gca_indexed(qd, kd, vd, idx.cuda(), wd, scale, **kw)
    o.backward(dout.cuda())
    return o, qd.grad, kd.grad, vd.grad, wd.grad


def test_bench_shape_whole_sequences_vs_oracle(lcm):
    """8 sequences x 256 chunks x 12 heads, K = 8, bf16 (the benchmark's problem: 12,288 kv-major
    and 12,240 q-major units on at most 148 CTAs, ~83 units per CTA).  Two whole sequences of the
    8-sequence GPU run are compared with the oracle, gradients included."""
    n, c, h, k = 8, 256, 12, 8
    q, kc, vc, idx, w, dout = cases.gca_indexed_case(100, n, c, h, k, dtype=torch.bfloat16)
    got = run(lcm, q, kc, vc, idx, w, dout)
    assert lcm.read_status() == 0
    for b in (0, 5):
        sl = slice(b, b + 1)
        ref = G.gca_indexed_grads(q[sl].float(), kc[sl].float(), vc[sl].float(), idx[sl], w[sl], 0.125, dout[sl].float())
        for name, g_, r_ in zip(NAMES, got, ref):
            g_b = g_[sl].reshape(r_.shape) if name in ("dk", "dv") else g_[sl]
            check(f"{name}[seq {b}]", g_b, r_, 2e-2)


@pytest.mark.parametrize("k", [16, 32])
def test_many_slots_per_unit(lcm, k):
    """K = 16 and 32 retrieved chunks per query chunk (ring stage = slot mod 6, two descriptor
    words per unit), 316 q-major units."""
    q, kc, vc, idx, w, dout = cases.gca_indexed_case(101 + k, 1, 80, 4, k, dtype=torch.bfloat16)
    got = run(lcm, q, kc, vc, idx, w, dout)
    ref = G.gca_indexed_grads(q.float(), kc.float(), vc.float(), idx, w, 0.125, dout.float())
    for name, g_, r_ in zip(NAMES, got, ref):
        check(name, g_.reshape(r_.shape), r_, 2e-2)
    assert lcm.read_status() == 0


@pytest.mark.parametrize("hq,hkv,n,c", [(8, 4, 2, 160), (8, 2, 4, 160), (4, 1, 4, 160)])
def test_grouped_query_heads_many_units(lcm, hq, hkv, n, c):
    """GQA 2, 4 and 4-with-one-kv-head through the indexed entry: q heads of a pair that share a kv
    head (one K/V tile for both), pairs that straddle two kv heads, and the kv-major pass summing
    the group's heads into one chunk gradient; >= 600 units per kernel."""
    g = torch.Generator().manual_seed(7 * hq + hkv)
    k = 4
    q = torch.randn(n, c - 1, hq, 64, 64, generator=g).bfloat16()
    kc = torch.randn(n, c, 64, hkv * 64, generator=g).bfloat16()
    vc = torch.randn(n, c, 64, hkv * 64, generator=g).bfloat16()
    idx, scores = cases.causal_indices(g, n, c, k)
    w = torch.nan_to_num(torch.softmax(scores, -1), nan=0.0)
    dout = torch.randn(n, c - 1, hq, 64, 64, generator=g).bfloat16()
    got = run(lcm, q, kc, vc, idx, w, dout)
    ref = G.gca_indexed_grads(q.float(), kc.float(), vc.float(), idx, w, 0.125, dout.float())
    for name, g_, r_ in zip(NAMES, got, ref):
        check(name, g_.reshape(r_.shape), r_, 2e-2)
    assert lcm.read_status() == 0


@pytest.mark.parametrize("h", [5, 1])
def test_odd_head_count_many_units(lcm, h):
    """An odd number of heads leaves the last unit of every (sequence, chunk) with ONE live head
    in its pair; 714 q-major units for h = 5."""
    n, c, k = 2, 120, 8
    q, kc, vc, idx, w, dout = cases.gca_indexed_case(110 + h, n, c, h, k, dtype=torch.bfloat16)
    got = run(lcm, q, kc, vc, idx, w, dout)
    ref = G.gca_indexed_grads(q.float(), kc.float(), vc.float(), idx, w, 0.125, dout.float())
    for name, g_, r_ in zip(NAMES, got, ref):
        check(name, g_.reshape(r_.shape), r_, 2e-2)
    assert lcm.read_status() == 0


@pytest.mark.parametrize("true_off_by_one", [False, True])
def test_cpu_reference_config_fp32(lcm, true_off_by_one):
    """The CPU-runnable configuration exactly: B = 2, H = 12, 64 chunks of 64 tokens (L = 4096),
    top-k = 8, float32, N(0,1) tensors, uniform causal indices, seed 0; once with the landmark row
    of K and V zeroed (how the model realises softmax-off-by-one, ``model/DRT.py:771-781``) and once
    with the explicit off-by-one softmax on un-zeroed caches.  1e-4 against the float64 oracle."""
    n, c, h, k = 2, 64, 12, 8
    q, kc, vc, idx, w, dout = cases.gca_indexed_case(0, n, c, h, k, dtype=torch.float32, zero_landmark=not true_off_by_one)
    ref = G.gca_indexed_grads(q, kc, vc, idx, w, 0.125, dout, work_dtype=torch.float64,
                              off_by_one=1.0 if true_off_by_one else 0.0)
    got = run(lcm, q, kc, vc, idx, w, dout, softmax_off_by_one=true_off_by_one)
    for name, g_, r_ in zip(NAMES, got, ref):
        check(name, g_.reshape(r_.shape), r_, 1e-4, rtol=1e-4, atol=1e-4)
    assert lcm.read_status() == 0
