"""Chunk-range-sharded retrieval and GCA decode over NCCL on 2+ GPUs (skipped on a 1-GPU box).

Each rank is a child process with its own GPU.  Every rank also runs the single-GPU kernels
over the whole cache on its own device and compares: the sharded selection must be
bit-identical (same packed keys, same indices), the weights equal, and the owner-computes
decode within bf16 tolerance of the one-GPU result (the partial outputs are summed in a
different order).
"""
import datetime
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _rank_main(rank, world, port, out):
    try:
        sys.path.insert(0, ROOT)
        sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
        import torch.distributed as dist
        import cases
        import long_context_modeling_b200 as lcm
        from long_context_modeling_b200 import sharded
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                                timeout=datetime.timedelta(seconds=60))
        report = {}
        for mode, head_dim in (("per_sequence", 0), ("per_head", 64)):
            e_total, topk, n = 4099, 8, 2
            lq, lk = cases.landmark_case(77, n, 1, e_total, d=768, std=0.125)
            lo, hi = sharded.shard_range(e_total, world, rank)
            got = sharded.sharded_lmk_topk(lq.to(dev), lk[:, lo:hi].contiguous().to(dev), topk, e_total=e_total,
                                           head_dim=head_dim)
            want = lcm.lmk_score_topk(lq.to(dev), lk.to(dev), topk, q_pos0=e_total - 1, head_dim=head_dim)
            lean = sharded.sharded_lmk_topk(lq.to(dev), lk[:, lo:hi].contiguous().to(dev), topk, e_total=e_total,
                                            head_dim=head_dim, validate=False)     # no header, no host checks
            report[mode] = (bool(torch.equal(got.keys, want.keys)) and bool(torch.equal(lean.keys, want.keys)),
                            bool(torch.equal(got.indices, want.indices)) and bool(torch.equal(lean.indices, want.indices)),
                            float((got.weights - want.weights).abs().max()))
        # owner-computes decode over a sharded K/V cache
        n, c, h, k = 2, 37, 4, 8
        g = torch.Generator().manual_seed(5)
        q = torch.randn(n, 1, h, 1, 64, generator=g).bfloat16()
        kc = torch.randn(n, c, 64, h * 64, generator=g).bfloat16()
        vc = torch.randn(n, c, 64, h * 64, generator=g).bfloat16()
        idx = torch.stack([torch.randperm(c, generator=g)[:k] for _ in range(n)]).view(n, 1, k)
        idx[0, 0, -1] = -1                                           # one padding slot
        w = torch.softmax(torch.randn(n, 1, k, generator=g), -1)
        w[0, 0, -1] = 0
        lo, hi = sharded.shard_range(c, world, rank)
        part = sharded.sharded_gca_decode(q.to(dev), kc[:, lo:hi].contiguous().to(dev), vc[:, lo:hi].contiguous().to(dev),
                                          idx.to(dev), w.to(dev), 0.125, e_total=c)
        whole = lcm.gca_indexed_nograd(q.to(dev), kc.to(dev), vc.to(dev), idx.to(dev), w.to(dev), 0.125)
        err = float((part.float() - whole.float()).abs().max() / whole.float().abs().max())
        report["decode_rel_err"] = err
        report["status"] = int(lcm.read_status())
        out.put((rank, "ok", report))
        dist.destroy_process_group()
    except Exception as exc:                      # surfaced by the parent
        out.put((rank, "error", repr(exc)))


def test_sharded_retrieval_and_decode_over_nccl():
    world = torch.cuda.device_count()
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    world = min(world, 4)
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29700 + os.getpid() % 200
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        item = out.get(timeout=300)
        results[item[0]] = item[1:]
    for p in procs:
        p.join(timeout=120)
    for r in range(world):
        assert results[r][0] == "ok", results
        rep = results[r][1]
        for mode in ("per_sequence", "per_head"):
            keys_eq, idx_eq, werr = rep[mode]
            assert keys_eq and idx_eq, (r, mode)
            assert werr <= 1e-6
        assert rep["decode_rel_err"] <= 2e-2
        assert rep["status"] == 0
