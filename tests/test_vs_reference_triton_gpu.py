"""The reference's OWN Triton GCA kernels, run on this GPU, as a second oracle.

``oracle/make_ref.py`` stages the reference's ``ltriton/gca.py`` (unchanged) under
``oracle/_ref/``; here its ``attention`` (``ltriton/gca.py:844``, forward + backward) and
``gca_kv_cache`` (``:846``, 2 and 1 query rows) run on the same seeded bf16 inputs as this
repository's drop-ins and must agree within the 2e-2 relative bound and the reference test's own
absolute tolerances (``ltriton/gca.py:938-961``: 1e-2 on out/dq/dk/dv, 0.5 on dw; ``:988,1011``).

If the file was not staged, or Triton cannot compile it for this GPU, the tests are skipped with
the reason; a numerical disagreement fails.
"""
import os
import sys

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lcm():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import long_context_modeling_b200 as m
    return m


@pytest.fixture(scope="module")
def ref():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import make_ref
    try:
        mod = make_ref.load()
    except FileNotFoundError:
        pytest.skip("oracle/_ref/ltriton_gca.py not staged (run oracle/make_ref.py next to a reference checkout)")
    except Exception as e:      # noqa: BLE001  (import-time failure of the reference file on this stack)
        pytest.skip(f"the reference Triton file does not import here: {type(e).__name__}: {e}")
    # one tiny call decides whether Triton can compile the kernels for this GPU
    try:
        q, k, v, w, _ = (t.cuda() for t in cases.gca_gathered_case(1, 2, 2, 2, 2, dtype=torch.bfloat16))
        mod.attention(q, k, v, w, 0.125, 0.0)
        torch.cuda.synchronize()
    except Exception as e:      # noqa: BLE001
        pytest.skip(f"Triton could not compile / run the reference kernels here: {type(e).__name__}: {str(e)[:300]}")
    return mod


def rel(a, b):
    a, b = a.detach().float(), b.detach().float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


@pytest.mark.parametrize("z,hq,hkv,k,std", [(24, 8, 2, 32, 0.5), (16, 12, 12, 8, 0.5), (6, 4, 2, 4, 1.0)])
def test_attention_fwd_bwd_matches_reference_triton(lcm, ref, z, hq, hkv, k, std):
    """The reference test's own recipe (GQA 4, K = 32, N(0, 0.5), weights = softmax(U)), the model's
    MHA 12/12 with K = 8, and a GQA 2 case with N(0, 1) inputs."""
    q, kk, v, w, dout = (t.cuda() for t in cases.gca_gathered_case(22, z, hq, hkv, k, std=std, dtype=torch.bfloat16))
    outs = []
    for fn in (ref.attention, lcm.attention):
        qd, kd, vd, wd = (t.clone().requires_grad_() for t in (q, kk, v, w))
        o = fn(qd, kd, vd, wd, 0.125, 0)
        o.backward(dout)
        outs.append((o, qd.grad, kd.grad, vd.grad, wd.grad))
    for name, r_, g_ in zip(("o", "dq", "dk", "dv", "dw"), *outs):
        assert g_.shape == r_.shape, name
        assert rel(g_, r_) <= 2e-2, (name, rel(g_, r_))
        atol = 0.5 if name == "dw" else 1e-2
        scale = max(1.0, r_.float().abs().max().item()) if std > 0.5 else 1.0
        assert (g_.float() - r_.float()).abs().max().item() <= atol * scale, name


@pytest.mark.parametrize("sq", [2, 1])
def test_gca_kv_cache_matches_reference_triton(lcm, ref, sq):
    """Decode shapes of the reference test: q rows 2 then 1, GQA 2, sm_scale 0.5."""
    q, kk, v, w, _ = (t.cuda() for t in cases.gca_gathered_case(30 + sq, 32, 8, 4, 8, s=sq, std=0.5, dtype=torch.bfloat16))
    with torch.no_grad():
        r_ = ref.gca_kv_cache(q, kk, v, w, 0.5, 0.0)
        g_ = lcm.gca_kv_cache(q, kk, v, w, 0.5, 0.0)
    assert g_.shape == r_.shape
    assert (g_.float() - r_.float()).abs().max().item() <= 1e-2
    assert rel(g_, r_) <= 2e-2


def test_eval_prefill_matches_reference_triton(lcm, ref):
    """Eval-mode prefill uses the inference kernel on full 64-row chunks (``model/DRT.py:379-382``)."""
    q, kk, v, w, _ = (t.cuda() for t in cases.gca_gathered_case(40, 20, 12, 12, 8, s=64, std=0.5, dtype=torch.bfloat16))
    with torch.no_grad():
        r_ = ref.gca_kv_cache(q, kk, v, w, 0.125, 0.0)
        g_ = lcm.gca_kv_cache(q, kk, v, w, 0.125, 0.0)
    assert (g_.float() - r_.float()).abs().max().item() <= 1e-2
    assert rel(g_, r_) <= 2e-2
