"""The allocation-free landmark top-k entry point, called through the C ABI.

Some hosts of this library are not allowed to obtain device scratch around a call: a server
whose memory pools own all of HBM, a plugin that lives inside another framework's allocator,
a loop that cannot afford an allocator call.  For them ``lmk_score_topk_static`` keeps its
per-block candidate lists in an array built into the library instead of a caller-provided
workspace.  This test drives it with ctypes exactly as such a host would and requires the
results to be identical to the regular entry point -- twice in a row with different problems,
because the built-in array is shared between calls and keeps its old contents.

The file name sorts last so that a run that stops at the first failure has already executed
every other test; the test does not depend on anything the other tests leave behind.
"""
import ctypes as C

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu


def _args(lib, lq, lk, k, outs, head_dim=0, splits=0, noise=None):
    keys, idx, sc, w, nv = outs
    a = lib.LmkTopkArgs()
    a.lmk_q, a.lmk_k = lq.data_ptr(), lk.data_ptr()
    a.out_keys, a.out_indices, a.out_scores = keys.data_ptr(), idx.data_ptr(), sc.data_ptr()
    a.out_weights, a.out_nvalid = w.data_ptr(), nv.data_ptr()
    a.q_batch_stride, a.q_row_stride = lq.stride(0), lq.stride(1)
    a.k_batch_stride, a.k_row_stride = lk.stride(0), lk.stride(1)
    n, cq, d = lq.shape
    e = lk.shape[1]
    a.q_pos0, a.e_base = e - cq, 0
    a.N, a.Cq, a.E, a.D, a.K = n, cq, e, d, k
    a.head_dim, a.score_round, a.splits = head_dim, 0, splits
    a.noise = noise.data_ptr() if noise is not None else None
    return a


def _outputs(rows_shape, k, dev):
    return (torch.full(rows_shape + (k,), -7, dtype=torch.int64, device=dev),
            torch.full(rows_shape + (k,), -7, dtype=torch.int32, device=dev),
            torch.full(rows_shape + (k,), -7.0, dtype=torch.float32, device=dev),
            torch.full(rows_shape + (k,), -7.0, dtype=torch.float32, device=dev),
            torch.full(rows_shape, -7, dtype=torch.int32, device=dev))


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from long_context_modeling_b200 import _lib as lib
    handle = lib.lib()
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: a decode-shaped scan with many splits, then a
    # batch-shaped one with per-head lists (the second reuses the array the first one filled)
    problems = [dict(seed=41, n=1, cq=1, e=40000, d=768, k=8, head_dim=0),
                dict(seed=42, n=2, cq=9, e=300, d=768, k=4, head_dim=0),
                dict(seed=43, n=1, cq=1, e=5000, d=768, k=8, head_dim=64),
                dict(seed=45, n=2, cq=5, e=400, d=768, k=8, head_dim=0, noise=True)]   # selection on noisy scores,
                                                                                    # noise-free scores recomputed
    for pb in problems:
        lq, lk = cases.landmark_case(pb["seed"], pb["n"], pb["cq"], pb["e"], d=pb["d"])
        lq, lk = lq.to(dev), lk.to(dev)
        rows_shape = (pb["n"], pb["cq"]) + ((pb["d"] // 64,) if pb["head_dim"] else ())
        noise = None
        if pb.get("noise"):
            g = torch.Generator().manual_seed(pb["seed"])
            noise = (-torch.empty(pb["n"], pb["cq"], pb["e"]).exponential_(generator=g).log()).to(dev)
        ref_out = _outputs(rows_shape, pb["k"], dev)
        a = _args(lib, lq, lk, pb["k"], ref_out, head_dim=pb["head_dim"], noise=noise)
        nbytes = handle.lmk_topk_workspace_bytes(C.byref(a))
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
        a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
        assert handle.lmk_score_topk(C.byref(a), stream) == 0
        got_out = _outputs(rows_shape, pb["k"], dev)
        b = _args(lib, lq, lk, pb["k"], got_out, head_dim=pb["head_dim"], noise=noise)      # no workspace at all
        assert handle.lmk_score_topk_static(C.byref(b), stream) == 0
        torch.cuda.synchronize()
        for name, r, g in zip(("keys", "indices", "scores", "weights", "n_valid"), ref_out, got_out):
            assert torch.equal(r, g), f"{name} differ for {pb}"
        assert int(ref_out[4].min()) >= 0          # outputs were really written


def test_static_scratch_entry_refuses_what_does_not_fit():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from long_context_modeling_b200 import _lib as lib
    handle = lib.lib()
    dev = torch.device("cuda", 0)
    lq, lk = cases.landmark_case(44, 1, 600, 600, d=768)
    lq, lk = lq.to(dev), lk.to(dev)
    outs = _outputs((1, 600), 32, dev)
    a = _args(lib, lq, lk, 32, outs, splits=8)       # 600 rows x 8 splits x 32 keys x 8 B = 1.2 MB > 1 MiB
    rc = handle.lmk_score_topk_static(C.byref(a), torch.cuda.current_stream().cuda_stream)
    assert rc == -10
    assert "1 MiB" in handle.gca_strerror(rc).decode()
    torch.cuda.synchronize()
    assert int(outs[1].max()) == -7                   # nothing was launched
    with pytest.raises(ValueError):
        lib.check(rc, "lmk_score_topk_static")
