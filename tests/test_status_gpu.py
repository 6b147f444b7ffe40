"""A bounded wait that expires must end as a STATUS, not as a hang.

Every spin-wait of the tensor-core kernels has an iteration limit; when it runs out the CTA
raises ``GCA_STATUS_TIMEOUT`` in the caller's status word, waits (bounded) for its copies in
flight, frees its tensor memory and returns, and the host turns the status into ``GcaError``.
This test builds a second copy of the library in which the forward's producer never requests
the first K tile of a CTA (``-DGCA_TEST_WITHHOLD_K``: a barrier that nothing completes; no
fault, no trap, no endless loop) with a short poll limit, runs one small forward in a child
process, and checks that the kernel returns, that the status says TIMEOUT, that
``check_status`` raises, and that the GPU context goes on working afterwards.
"""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_expired_wait_sets_status_and_host_raises(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from long_context_modeling_b200 import build
    lib = build.build_variant(str(tmp_path), ["-DGCA_TEST_WITHHOLD_K", "-DGCA_WAIT_LIMIT=20000"])
    code = textwrap.dedent(f"""
        import sys, torch
        sys.path.insert(0, {ROOT!r}); sys.path.insert(0, {os.path.join(ROOT, 'tests', 'golden')!r})
        import cases
        import long_context_modeling_b200 as lcm
        q, kc, vc, idx, w, _ = (t.cuda() for t in cases.gca_indexed_case(0, 1, 6, 2, 4, dtype=torch.bfloat16))
        out = lcm.gca_indexed_nograd(q, kc, vc, idx, w, 0.125, algo=2)
        torch.cuda.synchronize()                       # the kernel RETURNED
        bits = lcm.read_status(clear=False)
        print("status", bits)
        try:
            lcm.check_status()
            print("no error raised")
        except lcm.GcaError as e:
            print("raised", type(e).__name__)
        lcm.set_status_checks(True)                    # with checks on, the call itself raises
        try:
            lcm.gca_indexed_nograd(q, kc, vc, idx, w, 0.125, algo=2)
            print("second call: no error")
        except lcm.GcaError:
            print("second call raised")
        x = torch.ones(1024, device="cuda")
        print("context alive", float((x @ x).item()))
    """)
    env = dict(os.environ, GCA_B200_LIB=lib)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "status 2" in r.stdout, r.stdout
    assert "raised GcaError" in r.stdout
    assert "second call raised" in r.stdout
    assert "context alive 1024.0" in r.stdout
