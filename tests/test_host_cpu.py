"""Host-side checks that need no GPU: the C-ABI library loads and exports what the header
declares, argument validation returns error codes before any launch, the product path
refuses CPU tensors, and the sharded-retrieval exchange works (and fails loudly) across two
CPU ranks over gloo."""
import ctypes as C
import os
import re
import sys
import datetime

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from long_context_modeling_b200 import build, _lib
    build.build()
    return _lib


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "gca_b200.h")).read()
    body = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"^\s*(?:int|size_t|const char\*)\s+(\w+)\s*\(", body, flags=re.M))
    assert {"gca_fwd", "gca_bwd", "gca_decode", "lmk_score_topk", "lmk_topk_merge", "gca_cache_append",
            "gca_bwd_workspace_bytes", "lmk_topk_workspace_bytes", "gca_strerror", "gca_abi_version",
            "gca_sizeof"} <= declared
    handle = lib.lib()
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
    assert set(lib.EXPORTS) == declared
    assert handle.gca_abi_version() == lib.ABI_VERSION == 2


def test_struct_layouts_match(lib):
    handle = lib.lib()
    for which, st in enumerate((lib.GcaFwdArgs, lib.GcaBwdArgs, lib.LmkTopkArgs, lib.LmkMergeArgs, lib.CacheAppendArgs)):
        assert handle.gca_sizeof(which) == C.sizeof(st)


def _valid_fwd(lib):
    a = lib.GcaFwdArgs()
    for f in ("q", "k_cache", "v_cache", "indices", "weights", "out"):
        setattr(a, f, 0x10000)
    a.q_stride = lib.strides4(64 * 64 * 2, 64 * 64 * 2, 4096, 64)
    a.o_stride = lib.strides4(64 * 64 * 2, 64 * 64 * 2, 4096, 64)
    a.k_stride = lib.strides4(4 * 64 * 128, 64 * 128, 128, 64)
    a.v_stride = lib.strides4(4 * 64 * 128, 64 * 128, 128, 64)
    a.N, a.J, a.Hq, a.Hkv, a.S, a.L, a.D, a.K, a.C = 1, 1, 2, 2, 64, 64, 64, 4, 4
    a.dtype, a.algo, a.sm_scale, a.off_by_one = lib.BF16, 0, 0.125, 0.0
    return a


@pytest.mark.parametrize("mutate,code", [
    (lambda a: setattr(a, "q", None), -1),
    (lambda a: setattr(a, "out", None), -1),
    (lambda a: setattr(a, "dtype", 7), -2),
    (lambda a: setattr(a, "D", 128), -3),
    (lambda a: setattr(a, "L", 32), -3),
    (lambda a: setattr(a, "S", 65), -3),
    (lambda a: setattr(a, "K", 33), -3),
    (lambda a: setattr(a, "K", 0), -3),
    (lambda a: setattr(a, "Hkv", 3), -3),
    (lambda a: setattr(a, "sm_scale", 0.0), -3),
    (lambda a: setattr(a, "off_by_one", -1.0), -3),
    (lambda a: setattr(a, "q", 0x10004), -5),
    (lambda a: setattr(a, "k_stride", (C.c_int64 * 4)(4 * 64 * 128, 64 * 128, 100, 64)), -4),
    (lambda a: setattr(a, "algo", 9), -7),
])
def test_forward_argument_validation(lib, mutate, code):
    """Every rejected call returns its error code on the host, before any CUDA work."""
    a = _valid_fwd(lib)
    mutate(a)
    if code == -7:
        pytest.skip("algo is checked after validation succeeds, which would launch")
    assert lib.lib().gca_fwd(C.byref(a), None) == code
    assert lib.lib().gca_strerror(code).decode() != "unknown error"
    with pytest.raises(ValueError):
        lib.check(code, "gca_fwd")


def test_decode_and_topk_validation(lib):
    a = _valid_fwd(lib)
    a.S = 17
    assert lib.lib().gca_decode(C.byref(a), None) == -3
    t = lib.LmkTopkArgs()
    assert lib.lib().lmk_score_topk(C.byref(t), None) == -1
    t.lmk_q = t.lmk_k = t.out_keys = 0x10000
    t.N, t.Cq, t.E, t.D, t.K = 1, 1, 100, 770, 8
    assert lib.lib().lmk_score_topk(C.byref(t), None) == -3          # D not a multiple of 8
    t.D, t.K = 768, 40
    assert lib.lib().lmk_score_topk(C.byref(t), None) == -3
    t.K, t.head_dim = 8, 32
    assert lib.lib().lmk_score_topk(C.byref(t), None) == -3          # per-head mode needs head_dim 64
    t.head_dim = 0
    t.q_row_stride = t.k_row_stride = 768
    t.q_batch_stride, t.k_batch_stride = 768, 768 * 100
    assert lib.lib().lmk_score_topk(C.byref(t), None) == -6          # no workspace given
    assert lib.lib().lmk_topk_workspace_bytes(C.byref(t)) >= 8 * 8
    m = lib.LmkMergeArgs()
    assert lib.lib().lmk_topk_merge(C.byref(m), None) == -1
    c = lib.CacheAppendArgs()
    assert lib.lib().gca_cache_append(C.byref(c), None) == -1
    # a position beyond the destination's capacity is refused on the host (nothing is written)
    for f in ("new_k", "new_v", "k_cache", "v_cache"):
        setattr(c, f, 0x10000)
    c.N, c.count, c.pos, c.L, c.HD, c.Dm, c.dtype = 1, 3, 14, 64, 128, 0, lib.BF16
    c.new_batch_stride, c.cache_batch_stride = 3 * 64 * 128, 16 * 64 * 128
    c.capacity = 16
    assert lib.lib().gca_cache_append(C.byref(c), None) == -3          # chunks 14..16 of a 16-chunk buffer
    b = lib.GcaBwdArgs()
    assert lib.lib().gca_bwd(C.byref(b), None) == -1


def test_product_path_refuses_cpu_tensors_and_has_no_fallback(lib):
    import long_context_modeling_b200 as lcm
    q = torch.zeros(1, 1, 2, 64, 64, dtype=torch.bfloat16)
    kc = torch.zeros(1, 4, 64, 128, dtype=torch.bfloat16)
    idx = torch.zeros(1, 1, 4, dtype=torch.int64)
    w = torch.zeros(1, 1, 4)
    with pytest.raises(RuntimeError):
        lcm.gca_indexed(q, kc, kc, idx, w, 0.125)
    with pytest.raises(RuntimeError):
        lcm.lmk_score_topk(torch.zeros(1, 1, 768), torch.zeros(1, 4, 768), 2)
    with pytest.raises(RuntimeError):
        lcm.ChunkKVManager().append(torch.zeros(1, 1, 64, 128), torch.zeros(1, 1, 64, 128), torch.zeros(1, 1, 128))
    # nothing in the package imports the oracle
    pkg = os.path.join(ROOT, "long_context_modeling_b200")
    for fn in os.listdir(pkg):
        if fn.endswith(".py"):
            assert "oracle" not in open(os.path.join(pkg, fn)).read(), fn


def test_shard_ranges_cover_and_balance():
    from long_context_modeling_b200.sharded import shard_range
    for e in (1, 7, 8, 262144, 262145, 1000003):
        for g in (1, 2, 4, 8):
            spans = [shard_range(e, g, r) for r in range(g)]
            assert spans[0][0] == 0 and spans[-1][1] == e
            assert all(spans[i][1] == spans[i + 1][0] for i in range(g - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1


# ----------------------------------------------------------------------------------------
# two CPU ranks over gloo: exchange plumbing, merge equality, injected faults
# ----------------------------------------------------------------------------------------
def _oracle_score_fn(lq, lk, topk, q_pos0, e_base, head_dim=0):
    """Checker standing in for the CUDA scan on CPU ranks (tests only)."""
    sys.path.insert(0, ROOT)
    from oracle import retrieval_oracle as R
    from long_context_modeling_b200.retrieval import Retrieval
    n, cq, _ = lq.shape
    keys = np.zeros((n, cq, topk), dtype=np.uint64)
    for b in range(n):
        s = R.canonical_scores(lq[b].float().numpy(), lk[b].float().numpy())
        gidx = e_base + np.arange(s.shape[1], dtype=np.int64)
        k = R.pack_keys(s, np.broadcast_to(gidx, s.shape))
        vis = gidx[None, :] < (q_pos0 + np.arange(cq))[:, None]
        k = np.where(vis, k, np.uint64(0))
        srt = np.sort(k, axis=1)[:, ::-1][:, :topk]
        keys[b, :, :srt.shape[1]] = np.ascontiguousarray(srt)
    kt = torch.from_numpy(keys.view(np.int64))
    return Retrieval(kt, None, None, None, None)


def _oracle_merge_fn(keys, topk):
    from oracle import retrieval_oracle as R
    from long_context_modeling_b200.retrieval import Retrieval
    shape = keys.shape
    m = np.ascontiguousarray(R.merge_candidates(keys.numpy().view(np.uint64).reshape(-1, shape[-1]), topk))
    sc, idx = R.unpack_keys(m)
    return Retrieval(torch.from_numpy(m.view(np.int64)).reshape(shape[:-1] + (topk,)),
                     torch.from_numpy(idx).reshape(shape[:-1] + (topk,)), torch.from_numpy(sc), None, None)


def _rank_main(rank, world, port, mode, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import torch.distributed as dist
    import cases
    from long_context_modeling_b200 import sharded
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    e_total, topk = 203, 8
    lq, lk = cases.landmark_case(31, 2, 1, e_total, d=256)
    lo, hi = sharded.shard_range(e_total, world, rank)
    tamper = None
    if mode == "wrong_k" and rank == 1:
        tamper = lambda p: torch.cat([p[:2], torch.tensor([topk + 1]), p[3:]])
    if mode == "nan" and rank == 1:
        def tamper(p):
            p = p.clone()
            nan_key = (np.uint64(0xFFC00000) << np.uint64(32)) | np.uint64(0xFFFFFFFF - lo)
            p[sharded.HEADER] = int(np.array([nan_key]).view(np.int64)[0])
            return p
    if mode == "missing" and rank == 1:
        tamper = lambda p: torch.zeros_like(p)           # payload never filled in
    if mode == "foreign_index" and rank == 1:
        def tamper(p):
            p = p.clone()
            key = (np.uint64(0xC0000000) << np.uint64(32)) | np.uint64(0xFFFFFFFF - 0)   # chunk 0 is rank 0's
            p[sharded.HEADER] = int(np.array([key]).view(np.int64)[0])
            return p
    try:
        if mode == "absent" and rank == 1:
            out.put((rank, "left"))
            dist.destroy_process_group()
            return
        res = sharded.sharded_lmk_topk(lq, lk[:, lo:hi], topk, e_total=e_total, score_fn=_oracle_score_fn,
                                       merge_fn=_oracle_merge_fn, _tamper=tamper)
        out.put((rank, "ok", res.indices.tolist()))
    except sharded.ShardExchangeError as exc:
        out.put((rank, "error", str(exc)))
    finally:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


def _run_two_ranks(mode, port):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, mode, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(2):
        item = out.get(timeout=60)
        results[item[0]] = item[1:]
    for p in procs:
        p.join(timeout=60)
    return results


def test_sharded_topk_two_cpu_ranks_equals_single_scan():
    res = _run_two_ranks("ok", 29611)
    assert res[0][0] == "ok" and res[1][0] == "ok"
    assert res[0][1] == res[1][1], "every rank must hold the same merged result"
    import cases
    from oracle import retrieval_oracle as R
    lq, lk = cases.landmark_case(31, 2, 1, 203, d=256)
    for b in range(2):
        s = R.canonical_scores(lq[b].float().numpy(), lk[b].float().numpy())
        idx, _, _, _ = R.canonical_topk(s, R.visible_limit(1, 203), 8)
        assert res[0][1][b][0] == idx[0].tolist()


@pytest.mark.parametrize("mode,needle", [("wrong_k", "mismatch"), ("nan", "NaN"), ("missing", "magic"),
                                         ("foreign_index", "outside")])
def test_sharded_exchange_faults_are_detected_on_every_rank(mode, needle):
    port = 29620 + ["wrong_k", "nan", "missing", "foreign_index"].index(mode)
    res = _run_two_ranks(mode, port)
    for r in (0, 1):
        assert res[r][0] == "error", res
        assert needle in res[r][1] or "payload" in res[r][1]


def test_sharded_exchange_rank_absent_times_out_with_error():
    """A rank that leaves before the exchange: the survivor's collective ends with the
    group's timeout and surfaces as ShardExchangeError (no hang)."""
    res = _run_two_ranks("absent", 29630)
    assert res[1][0] == "left"
    assert res[0][0] == "error" and "exchange failed" in res[0][1]


def test_fused_ops_refuse_cpu_tensors_and_wrong_dtypes(lib):
    """The fused projections, the windowed decode attention and the fused LM-head loss exist on the GPU
    only: CPU tensors raise instead of taking another path, other dtypes are rejected."""
    import torch
    from long_context_modeling_b200 import fused_ops as F
    x = torch.zeros(4, 128, dtype=torch.bfloat16)
    w = torch.zeros(64, 128, dtype=torch.bfloat16)
    for call in (lambda: F.row_rms(x, 1e-5), lambda: F.linear(x, w), lambda: F.rmsnorm_linear(x, w, 1e-5),
                 lambda: F.linear_cross_entropy(x, w, torch.zeros(4, dtype=torch.int64)),
                 lambda: F.window_decode(torch.zeros(1, 1, 1, 64, dtype=torch.bfloat16), torch.zeros(1, 1, 8, 64, dtype=torch.bfloat16),
                                         torch.zeros(1, 1, 8, 64, dtype=torch.bfloat16), 4),
                 lambda: F.silu_mul(x),
                 lambda: F.window_ring_decode(torch.zeros(1, 1, 1, 64, dtype=torch.bfloat16), torch.zeros(1, 1, 8, 64, dtype=torch.bfloat16),
                                              torch.zeros(1, 1, 8, 64, dtype=torch.bfloat16), torch.zeros(1, 1, 64, dtype=torch.bfloat16),
                                              torch.zeros(1, 1, 64, dtype=torch.bfloat16), torch.zeros(1, dtype=torch.int64), 7)):
        with pytest.raises(RuntimeError):
            call()
    assert F.fold_gain(torch.ones(3, 4), torch.full((4,), 2.0)).dtype == torch.bfloat16
    assert float(F.fold_gain(torch.ones(3, 4), torch.full((4,), 2.0))[0, 0]) == 2.0


def test_nvtx_switch_and_call_helper(lib):
    lib.set_nvtx(False)
    with pytest.raises(ValueError):                      # a negative return code from the library -> ValueError
        lib.call("gca_linear", None, None)
