#!/usr/bin/env python
"""Benchmark of the GCA hot path: forward + backward of Grouped Cross-Attention read
straight from the chunk cache, at the DRT-16K shape (8 sequences x 16,384 positions per GPU,
12 heads x 64, chunk 64, top-k 8, bf16).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line (rank 0).  `value` = algorithmic TFLOP/s with inputs resident in HBM;
`e2e` = the same through the public Python API from pinned host buffers (every step's H2D and
D2H inside the timed region, overlapped across steps by `HostGcaPipeline`); `roofline` = the
slowest of the three tensor-core kernels against the measured dense bf16 peak (all three are
listed under `kernels`); `cpu_baseline` = the PyTorch einsum formulation the reference uses as its ground
truth (ltriton/gca.py:912-921 behind the gather of model/DRT.py:193-199) on the host cores.
Data are synthetic (seeded N(0,1) tensors, uniform causal retrieved ids) and stand in for the
PG19 / arXiv-math token data of the reference, which is not available offline.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

N_SEQ, CHUNKS, HEADS, TOPK, HEAD_DIM, CHUNK = 8, 256, 12, 8, 64, 64
FWD_FLOP_PER_SLOT = 4 * CHUNK * CHUNK * HEAD_DIM          # QK^T + PV for one (query chunk, head, slot)
FWD_BWD_FACTOR = 3.5                                      # backward counted as 2.5 x forward (ltriton/gca.py:1091-1092)
# dram__bytes_read.sum + dram__bytes_write.sum per launch, ncu capture of `--n-seq 2` (see profiles/)
TRAFFIC_2SEQ = {"fwd": 140.5e6 + 48.4e6, "bwd_kv": 265.2e6 + 71.5e6, "bwd_q": 211.6e6 + 83.0e6}


def valid_slots(chunks: int, topk: int) -> int:
    return sum(min(topk, j - 1) for j in range(1, chunks))


def workload_flops(n_seq: int) -> float:
    return float(n_seq * HEADS * valid_slots(CHUNKS, TOPK)) * FWD_FLOP_PER_SLOT


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def make_inputs(seed: int, n_seq: int, dtype=torch.bfloat16):
    """CPU tensors in the fixed order q, k_cache, v_cache, indices/scores, dout."""
    import cases
    return cases.gca_indexed_case(seed, n_seq, CHUNKS, HEADS, TOPK, dtype=dtype, zero_landmark=True)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._halt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.005)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


def bind_to_gpu_cpus(index: int) -> dict:
    """Restrict this process to the CPU cores that are local to GPU `index` (NVML's affinity mask,
    intersected with what the process may use), BEFORE any pinned host memory is allocated, so that
    the staging buffers land on the GPU's NUMA node.  Returns what was done, for the JSON line."""
    info = {"bound": False, "cpus": len(os.sched_getaffinity(0))}
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        local = {64 * i + b for i, wd in enumerate(words) for b in range(64) if (int(wd) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        want = local & allowed
        if want and want != allowed:
            os.sched_setaffinity(0, want)
            info = {"bound": True, "cpus": len(want), "of": len(allowed)}
        elif want:
            info["note"] = "every allowed core is local to the GPU"
    except Exception as e:                       # no NVML, no affinity call: run unbound and say so
        info["note"] = f"not bound: {type(e).__name__}"
    return info


# --------------------------------------------------------------------------------------------
# CPU arms (the oracle is only ever the thing measured here as the *baseline*, never the product)
# --------------------------------------------------------------------------------------------
def cpu_reference_step(sample):
    from oracle import gca_oracle as G
    q, kc, vc, idx, w, dout = sample
    G.gca_indexed_grads(q, kc, vc, idx, w, 1.0 / 8.0, dout, work_dtype=torch.float32)


def run_cpu(steps: int, warmup: int, n_seq_sample: int):
    torch.set_num_threads(os.cpu_count() or 1)
    sample = tuple(t.float() if t.is_floating_point() else t for t in make_inputs(0, n_seq_sample, torch.float32))
    for _ in range(warmup):
        cpu_reference_step(sample)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_reference_step(sample)
    dt = (time.perf_counter() - t0) / steps
    return workload_flops(n_seq_sample) * FWD_BWD_FACTOR / dt / 1e12, dt


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 5)), max(1, min(args.warmup, 2))
    tflops, dt = run_cpu(steps, warmup, 1)
    cores = os.cpu_count() or 1
    sample = f"1 of the {N_SEQ} sequences per step (256 chunks x 12 heads x top-8, fp32), {steps} steps"
    line = {"impl": "reference", "metric": "gca_fwd_bwd_tflops", "value": tflops, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_dict(),
            "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def config_dict():
    return {"workload": "GCA fwd+bwd at the DRT-16K shape: 8 sequences x 256 chunks x 64 positions per GPU, "
                        "12 heads x 64, top-k 8, chunk cache read by retrieved index, bf16 (BASELINE configs[1] "
                        "hot path == configs[2] point L=16K, K=8, BxH=96)",
            "n_seq_per_gpu": N_SEQ, "chunks": CHUNKS, "heads": HEADS, "head_dim": HEAD_DIM, "topk": TOPK,
            "valid_slots_per_seq_head": valid_slots(CHUNKS, TOPK),
            "cache_policy": "inputs (q, caches, dout: ~0.8 GB per step) exceed the 126 MB L2; two input sets alternate",
            "parallelism": "one process per GPU, sequences sharded over ranks, no data-path collective"}


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
def gpu_arm(args):
    import torch.distributed as dist
    import long_context_modeling_b200 as lcm
    from long_context_modeling_b200 import gca as gmod

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the GCA path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    binding = bind_to_gpu_cpus(physical_gpu_index(local))      # before the pinned buffers exist
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    scale = 1.0 / 8.0

    # two alternating input sets (different seeds per rank: independent sequences, weak scaling)
    host_sets = []
    for s in range(2):
        q, kc, vc, idx, w, dout = make_inputs(1000 * rank + s, N_SEQ)
        host_sets.append(tuple(t.pin_memory() for t in (q, kc, vc, idx.to(torch.int32), w, dout)))
    dev_sets = [tuple(t.to(dev) for t in hs) for hs in host_sets]

    def device_step(ds):
        q, kc, vc, idx, w, dout = ds
        q = q.detach().requires_grad_()
        kc = kc.detach().requires_grad_()
        vc = vc.detach().requires_grad_()
        w = w.detach().requires_grad_()
        o = lcm.gca_indexed(q, kc, vc, idx, w, scale)
        o.backward(dout)
        return o, q.grad, kc.grad, vc.grad, w.grad

    pipe = lcm.HostGcaPipeline(dev, scale, depth=3)
    e2e_check = [0.0]

    def e2e_step(hs):
        done = pipe.submit(hs)
        if done is not None:
            e2e_check[0] += float(done[4][0, 1, 0])          # the host reads the finished step's result

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, sets, steps, warmup, finish=None):
        for i in range(warmup):
            fn(sets[i % 2])
        if finish:
            finish()
        barrier()
        sampler = ClockSampler(physical_gpu_index(local))
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(sets[i % 2])
        if finish:
            finish()                      # waits for the last downloads: they are part of the timed region
        e1.record()
        barrier()
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, clocks

    steps, warmup = args.steps, max(3, args.warmup)
    ms_dev, clocks = timed(device_step, dev_sets, steps, warmup)
    ms_e2e, _ = timed(e2e_step, host_sets, max(6, steps // 2), 4, finish=pipe.drain)

    # The host ceiling of the end-to-end step: one step's upload and download bytes moved with no
    # kernel at all, every rank at the same time (the ranks share the host's memory and PCIe root
    # complexes): upload alone, download alone, both directions at once.
    up_dst = [torch.empty_like(t, device=dev) for t in host_sets[0]]
    dn_src = torch.empty(pipe.d2h_bytes, dtype=torch.uint8, device=dev)
    dn_dst = torch.empty(pipe.d2h_bytes, dtype=torch.uint8).pin_memory()
    s_up, s_dn = torch.cuda.Stream(), torch.cuda.Stream()

    def copies(up, down):
        def run(_):
            if up:
                with torch.cuda.stream(s_up):
                    for d, h in zip(up_dst, host_sets[0]):
                        d.copy_(h, non_blocking=True)
            if down:
                with torch.cuda.stream(s_dn):
                    dn_dst.copy_(dn_src, non_blocking=True)
            torch.cuda.current_stream().wait_stream(s_up)
            torch.cuda.current_stream().wait_stream(s_dn)
        return run
    ms_up = timed(copies(True, False), host_sets, 5, 3)[0]
    ms_dn = timed(copies(False, True), host_sets, 5, 3)[0]
    ms_both = timed(copies(True, True), host_sets, 5, 3)[0]
    del up_dst, dn_src, dn_dst

    # the three tensor-core kernels one at a time (one launch per call), for the roofline
    def time_calls(fn, reps):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    reps = max(10, steps)
    fwd_out = [gmod.gca_forward_with_lse(*ds[:5], scale) for ds in dev_sets]
    ms_fwd = time_calls(lambda i: gmod.gca_forward_with_lse(*dev_sets[i % 2][:5], scale), reps)
    bufs = []
    for ds, (_, lse) in zip(dev_sets, fwd_out):          # inverse index once per input set, then the stages alone
        bufs.append(gmod.gca_backward_stages(*ds[:5], ds[5], lse, scale, stages=gmod.BWD_STAGE_INDEX))

    def stage(i, which):
        ds = dev_sets[i % 2]
        gmod.gca_backward_stages(*ds[:5], ds[5], fwd_out[i % 2][1], scale, stages=which, bufs=bufs[i % 2])

    ms_idx = time_calls(lambda i: stage(i, gmod.BWD_STAGE_INDEX), reps)
    ms_q = time_calls(lambda i: stage(i, gmod.BWD_STAGE_Q), reps)      # first: it writes the per-row terms the kv-major pass reads
    ms_kv = time_calls(lambda i: stage(i, gmod.BWD_STAGE_KV), reps)
    status = lcm.read_status()

    flops_fwd = workload_flops(N_SEQ)
    flops_step = flops_fwd * FWD_BWD_FACTOR
    value = flops_step * world / (ms_dev * 1e-3) / 1e12
    e2e_val = flops_step * world / (ms_e2e * 1e-3) / 1e12
    peak = peaks["bf16_tflops"]
    # Algorithmic work per kernel, in units of the forward's two products (S = QK^T, O = PV):
    # dK/dV kernel = dV + dK (its recomputed S and dP are overhead, not counted), dQ kernel =
    # S + dP + dQ, so that forward + both = 3.5 x forward, the convention of the headline metric.
    # DRAM traffic per launch: dram__bytes_read + dram__bytes_write of one ncu capture of the
    # 2-sequence case (profiles/), scaled by the number of sequences (traffic grows with units).
    kernels = {}
    for name, ms, work, traffic_2seq in (("fwd_tc_kernel", ms_fwd, 1.0, TRAFFIC_2SEQ["fwd"]),
                                         ("bwd_kv_tc_kernel", ms_kv, 1.0, TRAFFIC_2SEQ["bwd_kv"]),
                                         ("bwd_q_tc_kernel (+ dw reduction)", ms_q, 1.5, TRAFFIC_2SEQ["bwd_q"])):
        ach = flops_fwd * work / (ms * 1e-3) / 1e12
        kernels[name] = {"ms": ms, "algorithmic_flops_per_launch": flops_fwd * work, "achieved_tflops": ach,
                         "frac_of_peak": ach / peak, "dram_traffic_bytes_per_launch": traffic_2seq * N_SEQ / 2}
    kernels["inverse index (csr_small_kernel; incl. ~30 us of host launch path)"] = {"ms": ms_idx}
    top = max((k for k in kernels if "ms" in kernels[k] and "achieved_tflops" in kernels[k]), key=lambda k: kernels[k]["ms"])
    line = {
        "metric": "gca_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_dev, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": config_dict(), "clocks": clocks,
        "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": pipe.h2d_bytes,
                "d2h_bytes_per_step": pipe.d2h_bytes, "ms_per_step": ms_e2e,
                "how": "HostGcaPipeline, 3 steps in flight: upload, kernels and download of consecutive steps overlap",
                "host_ceiling": {"what": "one step's bytes copied with no kernel running, all ranks at once, max over ranks",
                                 "h2d_gbs_per_gpu": pipe.h2d_bytes / (ms_up * 1e-3) / 1e9,
                                 "d2h_gbs_per_gpu": pipe.d2h_bytes / (ms_dn * 1e-3) / 1e9,
                                 "both_directions_ms": ms_both,
                                 "ceiling_value": flops_step * world / (ms_both * 1e-3) / 1e12,
                                 "e2e_frac_of_ceiling": ms_both / ms_e2e},
                "host_binding": binding},
        "gpu_launches": 5 * steps,      # fwd_tc, csr_small, bwd_kv_tc, bwd_q_tc, dw_reduce
        "kernels": kernels,
        "roofline": {"kernel": top, "bound": "tensor", "achieved": kernels[top]["achieved_tflops"],
                     "peak": peak, "unit": "TFLOP/s", "frac": kernels[top]["frac_of_peak"],
                     "peak_source": peaks["source"] + " burst dense bf16",
                     "traffic": kernels[top]["dram_traffic_bytes_per_launch"],
                     "algorithmic_flops_per_launch": kernels[top]["algorithmic_flops_per_launch"],
                     "pct_of_tensor_peak_fwd_bwd": 100.0 * value / world / peak},
        "device_status": status,
    }
    if rank == 0 and world == 1 and not args.no_cpu:
        tf, dt = run_cpu(2, 1, 1)
        line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": os.cpu_count() or 1, "kind": "port",
                                "sample": "1 of the 8 sequences (256 chunks x 12 heads x top-8), fp32 einsum + "
                                          "gather + autograd, 2 timed steps"}
    if world > 1:
        # the path that DOES exchange data between GPUs: 16M-token landmark retrieval over a cache
        # sharded by chunk range (both scoring modes), so that multi-GPU runs of the default line
        # carry it
        del dev_sets, fwd_out, bufs
        torch.cuda.empty_cache()
        sub = {}
        for mode, per_head in (("per_sequence", False), ("per_head", True)):
            r = measure_retrieval(dev, world, rank, local, per_head, 100, 10, peaks)
            sub[mode] = {"n_gpu_us": r["ms_per_step"] * 1e3, "n_gpu_eager_us": (r["eager_ms_per_step"] or 0) * 1e3,
                         "local_scan_us": r["roofline"]["us_per_launch"], "local_scan_gbs_per_gpu": r["roofline"]["achieved"],
                         "local_scan_frac_of_hbm_peak": r["roofline"]["frac"], "whole_cache_gbs": r["value"],
                         "sharded_gca_decode_us": None if r.get("sharded_gca_decode_ms_per_step") is None
                         else r["sharded_gca_decode_ms_per_step"] * 1e3}
        line["retrieval"] = {"what": "landmark top-8 over 262,144 cached chunks (16M tokens), batch 1, cache sharded by chunk "
                                     "range over the ranks; CUDA-graph replay of the local scan + the fused peer-store exchange and merge kernel, "
                                     "max over ranks (n_gpu_eager_us: the NCCL all-gather path issued from Python)",
                             **sub}
    if rank == 0 and world == 1 and args.triton_ref:
        del dev_sets, fwd_out, bufs
        torch.cuda.empty_cache()
        line["reference_triton_gpu"] = run_triton_ref_subprocess(N_SEQ)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------------
# The reference's own Triton kernels on this GPU (a GPU-vs-GPU anchor beside the CPU baseline)
# --------------------------------------------------------------------------------------------
def triton_ref_arm(args):
    """Times the reference's unmodified Triton GCA (`ltriton/gca.py`: `attention` = `_attention.apply`,
    line 844), staged under oracle/_ref by oracle/make_ref.py, at the same workload: the K/V chunks
    are first gathered and laid out as the reference model does (`model/DRT.py:193-199,321-332`),
    then `attention` forward and forward + backward are timed with CUDA events.  Prints one JSON
    object; on any failure the object carries `unavailable` with the reason."""
    out = {"impl": "reference_triton", "what": "ltriton/gca.py attention fwd / fwd+bwd on pre-gathered chunks, same inputs"}
    try:
        import triton
        out["triton"] = triton.__version__
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import make_ref
        from oracle import gca_oracle as G
        mod = make_ref.load()
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(0)
        n_seq = args.n_seq
        q, kc, vc, idx, w, dout = (t.to(dev) for t in make_inputs(0, n_seq))
        z = n_seq * (CHUNKS - 1)

        def ev_time(fn, reps):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / reps

        gather = lambda: G.gather_chunks(kc, vc, idx, HEADS)     # noqa: E731  (advanced-index gather + head split + contiguous)
        ms_gather = ev_time(gather, 5)
        gk, gv = gather()
        gk, gv = gk.contiguous().requires_grad_(), gv.contiguous().requires_grad_()
        qz = q.reshape(z, HEADS, CHUNK, HEAD_DIM).contiguous().requires_grad_()
        wz = torch.where(idx < 0, torch.zeros_like(w), w).reshape(z, TOPK).contiguous().requires_grad_()
        dz = dout.reshape(z, HEADS, CHUNK, HEAD_DIM).contiguous()
        scale = 1.0 / 8.0
        ms_fwd = ev_time(lambda: mod.attention(qz, gk, gv, wz, scale, 0.0), 10)

        def fwd_bwd():
            o = mod.attention(qz, gk, gv, wz, scale, 0.0)
            o.backward(dz)
            qz.grad = gk.grad = gv.grad = wz.grad = None
        ms_step = ev_time(fwd_bwd, 10)
        flops = workload_flops(n_seq)
        out.update({"n_seq": n_seq, "gather_ms": ms_gather, "fwd_ms": ms_fwd, "fwd_bwd_ms": ms_step,
                    "fwd_tflops": flops / (ms_fwd * 1e-3) / 1e12,
                    "fwd_bwd_tflops": flops * FWD_BWD_FACTOR / (ms_step * 1e-3) / 1e12,
                    "fwd_bwd_with_gather_tflops": flops * FWD_BWD_FACTOR / ((ms_step + ms_gather) * 1e-3) / 1e12,
                    "note": "backward excludes the scatter-add of the gathered dK/dV into the cache that the model's autograd adds"})
    except BaseException as e:      # noqa: BLE001
        out["unavailable"] = f"{type(e).__name__}: {str(e)[:400]}"
    print(json.dumps(out), flush=True)


def run_triton_ref_subprocess(n_seq: int, timeout_s: int = 420):
    """The Triton leg in a process of its own (its JIT, autotuner and 8 GB of gathered tensors stay
    out of this process), bounded in time."""
    import subprocess
    if not os.path.isfile(os.path.join(ROOT, "oracle", "_ref", "ltriton_gca.py")):
        return {"unavailable": "oracle/_ref/ltriton_gca.py not staged"}
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        env.pop(k, None)
    try:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--workload", "triton-ref", "--n-seq", str(n_seq)],
                           capture_output=True, text=True, timeout=timeout_s, env=env)
        for ln in reversed(r.stdout.strip().splitlines()):
            if ln.startswith("{"):
                return json.loads(ln)
        return {"unavailable": f"no output (exit {r.returncode}): {r.stderr[-300:]}"}
    except subprocess.TimeoutExpired:
        return {"unavailable": f"did not finish within {timeout_s} s"}


# --------------------------------------------------------------------------------------------
# Secondary workloads (not the default line): the HBM-bound kernels either side of GCA
# --------------------------------------------------------------------------------------------
def _graph_time(fn, flush, inner=10, reps=15):
    """Device time per call with host launch overhead removed: `inner` calls captured in one
    CUDA graph, an L2 flush between replays, median over `reps`.  `fn` may be a list of `inner`
    callables (calls that read different data, so that no call finds its input in L2)."""
    fns = fn if isinstance(fn, (list, tuple)) else [fn] * inner
    inner = len(fns)
    for f in fns[:3]:
        f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns:
            f()
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / inner)
    return statistics.median(ts)


def measure_retrieval(dev, world, rank, local, per_head, steps, warmup, peaks, with_cpu=False):
    """Landmark scoring + top-k over 262,144 cached chunks (a 16M-token context), batch 1: the
    decode-time retrieval block (model/DRT.py:825-849).  With N GPUs the cache is sharded by chunk
    range (strong scaling): local scan, one all-gather of the packed candidates, merge -- replayed
    from a CUDA graph (`ShardedRetriever`), and eager for comparison.  Returns the JSON line."""
    import torch.distributed as dist
    import long_context_modeling_b200 as lcm
    from long_context_modeling_b200 import sharded
    e_total, d, topk = 262144, 768, 8
    head_dim = 64 if per_head else 0
    lo, hi = sharded.shard_range(e_total, world, rank)
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    lk = (torch.randn(1, hi - lo, d, generator=g, device=dev) * 0.125).bfloat16()
    gq = torch.Generator().manual_seed(7)
    lq_host = (torch.randn(1, 1, d, generator=gq) * 0.125).bfloat16().pin_memory()
    lq = lq_host.to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    exchange = sharded.PeerExchange(dev, max_rows=16) if world > 1 else None
    retriever = (sharded.ShardedRetriever(lq, lk, topk, e_total=e_total, exchange=exchange, head_dim=head_dim)
                 if world > 1 else None)

    def step():
        if world == 1:
            return lcm.lmk_score_topk(lq, lk, topk, head_dim=head_dim)
        return retriever(lq)

    def eager_step():
        return sharded.sharded_lmk_topk(lq, lk, topk, e_total=e_total, head_dim=head_dim, validate=False)

    def e2e_step():
        q = lq_host.to(dev, non_blocking=True)
        r = lcm.lmk_score_topk(q, lk, topk, head_dim=head_dim) if world == 1 else retriever(q)
        return r.indices.cpu(), r.weights.cpu()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        sampler = ClockSampler(physical_gpu_index(local))
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, clocks

    ms, clocks = timed(step, steps, warmup)
    ms_e2e, _ = timed(e2e_step, steps, warmup)
    ms_eager = timed(eager_step, steps, warmup)[0] if world > 1 else None            # NCCL all-gather + merge, issued from Python
    ms_p2p_eager = (timed(lambda: sharded.sharded_lmk_topk(lq, lk, topk, e_total=e_total, head_dim=head_dim, exchange=exchange),
                          steps, warmup)[0] if world > 1 else None)
    # GCA decode over the winners with the K/V cache sharded the same way: every rank attends over the
    # retrieved chunks it owns, the (1, 12, 1, 64) partial outputs are summed with one all-reduce
    ms_gca = None
    if world > 1 and not per_head:
        kv_shard = [torch.empty(1, hi - lo, 64, d, dtype=torch.bfloat16, device=dev).normal_(generator=g) for _ in range(2)]
        qd = torch.randn(1, 1, d // 64, 1, 64, generator=g, device=dev).bfloat16()
        won = retriever(lq)
        gi, gw = won.indices.view(1, 1, topk).clone(), won.weights.view(1, 1, topk).clone()
        ms_gca = timed(lambda: sharded.sharded_gca_decode(qd, kv_shard[0], kv_shard[1], gi, gw, 0.125, e_total=e_total), steps, warmup)[0]
        del kv_shard
    # the scan + finalize kernels of this rank alone, launch overhead removed
    ms_scan = _graph_time(lambda: lcm.lmk_score_topk(lq, lk, topk, head_dim=head_dim), flush)
    bytes_total = e_total * d * 2
    bytes_local = (hi - lo) * d * 2
    achieved = bytes_local / (ms_scan * 1e-3) / 1e9
    line = {"metric": "lmk_topk_scan_gbs", "value": bytes_total / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16 in, f32 scores, u64 keys", "data": "synthetic",
            "config": {"workload": "landmark score + causal mask + top-8 + weights over 262,144 cached chunks "
                                   "(16M-token context), batch 1, " + ("per-head 64-d scores" if head_dim else
                                                                          "per-sequence 768-d scores"),
                       "landmarks": e_total, "hidden": d, "topk": topk, "per_head": bool(head_dim),
                       "cache_policy": "the landmark cache (403 MB / n_gpus per GPU) exceeds the 126 MB L2 at N <= 2; "
                                       "the graph-timed kernel figure flushes L2 between replays",
                       "parallelism": "cache sharded by chunk range; candidates exchanged by peer stores into every rank's mailbox "
                                      "and merged in the same kernel (one launch per rank); scan + exchange replayed from a CUDA "
                                      "graph; eager times (NCCL all-gather path, peer-exchange path) reported beside it"},
            "clocks": clocks,
            "e2e": {"value": bytes_total / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": lq_host.numel() * 2,
                    "d2h_bytes_per_step": topk * 8 * (d // 64 if head_dim else 1), "ms_per_step": ms_e2e},
            "eager_ms_per_step": ms_eager, "eager_peer_exchange_ms_per_step": ms_p2p_eager,
            "sharded_gca_decode_ms_per_step": ms_gca,      # owner-computes decode over the sharded K/V cache + all-reduce, eager
            "gpu_launches": (2 if world == 1 else 3) * steps,      # scan, finalize (+ exchange-and-merge)
            "roofline": {"kernel": "lmk_scan_kernel + lmk_finalize_kernel", "bound": "hbm", "achieved": achieved,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "peak_source": peaks["source"] + " copy bandwidth", "traffic": None,
                         "algorithmic_bytes_per_launch": bytes_local, "us_per_launch": ms_scan * 1e3},
            "device_status": lcm.read_status()}
    if with_cpu:
        torch.set_num_threads(os.cpu_count() or 1)
        lkc, lqc = lk.float().cpu(), lq.float().cpu()
        t0 = time.perf_counter()
        reps = 10
        for _ in range(reps):
            sc = torch.einsum("nqd,ned->nqe", lqc, lkc) / d ** 0.5
            torch.softmax(torch.topk(sc, topk, dim=-1).values, -1)
        dt = (time.perf_counter() - t0) / reps
        line["cpu_baseline"] = {"value": bytes_total / dt / 1e9, "unit": "GB/s", "cores": os.cpu_count() or 1, "kind": "port",
                                "sample": f"the full 262,144 x 768 scan in fp32 (einsum + topk + softmax), {reps} queries"}
    torch.cuda.synchronize()
    del retriever
    if exchange is not None:
        exchange.close()
    del lk, flush
    torch.cuda.empty_cache()
    return line


def retrieval_arm(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    line = measure_retrieval(dev, world, rank, local, args.per_head, max(args.steps, 50), max(5, args.warmup), load_peaks(),
                             with_cpu=(rank == 0 and world == 1 and not args.no_cpu))
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def decode_arm(args):
    """GCA for one generated token: 32 sequences, 12 heads, 8 retrieved chunks each read from a
    1,024-chunk cache (ltriton/gca.py:846-888 with q of one row).  Independent sequences: with N
    GPUs each holds 32 sequences of its own (weak scaling)."""
    import torch.distributed as dist
    import long_context_modeling_b200 as lcm
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    n, c, h, k = 32, 1024, 12, 8
    g = torch.Generator(device=dev).manual_seed(99 + rank)
    kc = torch.randn(n, c, 64, h * 64, generator=g, device=dev, dtype=torch.bfloat16)
    vc = torch.randn(n, c, 64, h * 64, generator=g, device=dev, dtype=torch.bfloat16)
    q = torch.randn(n, 1, h, 1, 64, generator=g, device=dev, dtype=torch.bfloat16)
    idx_sets = [torch.stack([torch.randperm(c, device=dev)[:k] for _ in range(n)]).view(n, 1, k).int() for _ in range(10)]
    idx = idx_sets[0]
    w = torch.softmax(torch.randn(n, 1, k, device=dev), -1)
    q_host, idx_host, w_host = q.cpu().pin_memory(), idx.cpu().pin_memory(), w.cpu().pin_memory()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    calls = [0]

    def step():                                  # ten index sets in turn: 503 MB of distinct tiles, 4 x the L2
        calls[0] += 1
        return lcm.gca_indexed_nograd(q, kc, vc, idx_sets[calls[0] % 10], w, 0.125)

    def e2e_step():
        o = lcm.gca_indexed_nograd(q_host.to(dev, non_blocking=True), kc, vc, idx_host.to(dev, non_blocking=True),
                                   w_host.to(dev, non_blocking=True), 0.125)
        return o.cpu()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(physical_gpu_index(local))
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, clocks

    steps, warmup = max(args.steps, 100), max(5, args.warmup)
    ms, clocks = timed(step, steps, warmup)
    ms_e2e, _ = timed(e2e_step, steps, warmup)
    ms_k = _graph_time([(lambda s=s: lcm.gca_indexed_nograd(q, kc, vc, s, w, 0.125)) for s in idx_sets], flush)
    nbytes = n * h * k * 2 * 64 * 64 * 2
    achieved = nbytes / (ms_k * 1e-3) / 1e9
    line = {"metric": "gca_decode_gbs", "value": nbytes * world / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "GCA decode, one query row: 32 sequences x 12 heads x 8 retrieved chunks out of 1,024 "
                                   "(50.3 MB of K/V tiles per call)", "sequences": n, "chunks": c, "heads": h, "topk": k,
                       "cache_policy": "6.4 GB of caches per GPU; ten index sets in turn (503 MB of distinct tiles, 4 x the L2) "
                                       "and an L2 flush between graph replays, so every call reads its tiles from HBM",
                       "parallelism": "independent sequences per GPU, no collective"},
            "clocks": clocks,
            "e2e": {"value": nbytes * world / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": q_host.numel() * 2 + idx_host.numel() * 4 + w_host.numel() * 4,
                    "d2h_bytes_per_step": q_host.numel() * 2, "ms_per_step": ms_e2e},
            "gpu_launches": steps,
            "roofline": {"kernel": "decode_rows_kernel", "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"] + " copy bandwidth",
                         "traffic": None, "algorithmic_bytes_per_launch": nbytes, "us_per_launch": ms_k * 1e3},
            "device_status": lcm.read_status()}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def window_decode_arm(args):
    """Sliding-window ALiBi attention of one decode step (the reference's flash_attn_with_kvcache call,
    model/llama.py:684-688): 32 sequences x 12 heads, one new position against 513 cached keys per
    head, one layer.  HBM-bound; ten caches in turn and an L2 flush between graph replays."""
    import long_context_modeling_b200 as lcm
    from long_context_modeling_b200 import fused_ops as F
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    n, h, t, window = 32, 12, 513, 512
    g = torch.Generator(device=dev).manual_seed(3)
    ks = [torch.randn(n, h, t, 64, generator=g, device=dev).bfloat16() for _ in range(10)]
    vs = [torch.randn(n, h, t, 64, generator=g, device=dev).bfloat16() for _ in range(10)]
    q = torch.randn(n, h, 1, 64, generator=g, device=dev).bfloat16()
    q_host = q.cpu().pin_memory()
    slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / h) for i in range(h)], device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    calls = [0]

    def step():
        calls[0] += 1
        return F.window_decode(q, ks[calls[0] % 10], vs[calls[0] % 10], window, slopes, 0.125)

    def e2e_step():
        calls[0] += 1
        return F.window_decode(q_host.to(dev, non_blocking=True), ks[calls[0] % 10], vs[calls[0] % 10], window, slopes, 0.125).cpu()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        sampler = ClockSampler(physical_gpu_index(0))
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps, sampler.stop()

    steps, warmup = max(args.steps, 100), max(5, args.warmup)
    ms, clocks = timed(step, steps, warmup)
    ms_e2e, _ = timed(e2e_step, steps, warmup)
    ms_k = _graph_time([(lambda i=i: F.window_decode(q, ks[i], vs[i], window, slopes, 0.125)) for i in range(10)], flush)
    # the ring form the fused token step uses: the new K / V row replaces the oldest row inside the same kernel
    kn, vn = torch.randn(n, h, 64, generator=g, device=dev).bfloat16(), torch.randn(n, h, 64, generator=g, device=dev).bfloat16()
    count = torch.full((1,), 100, dtype=torch.int64, device=dev)
    ms_ring = _graph_time([(lambda i=i: F.window_ring_decode(q, ks[i], vs[i], kn, vn, count, window, slopes, 0.125)) for i in range(10)], flush)
    nbytes = 2 * n * h * t * 128
    achieved = nbytes / (ms_k * 1e-3) / 1e9
    line = {"metric": "window_decode_gbs", "value": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": 1, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "sliding-window (512) causal attention with ALiBi, one new position: 32 sequences x 12 heads "
                                   "x 513 cached keys (50.4 MB of K/V per call), one layer", "sequences": n, "heads": h, "keys": t,
                       "cache_policy": "ten caches in turn (504 MB, 4 x the L2) and an L2 flush between graph replays"},
            "clocks": clocks,
            "e2e": {"value": nbytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": q_host.numel() * 2,
                    "d2h_bytes_per_step": q_host.numel() * 2, "ms_per_step": ms_e2e},
            "gpu_launches": steps,
            "roofline": {"kernel": "win_decode_kernel", "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"] + " copy bandwidth", "traffic": None,
                         "algorithmic_bytes_per_launch": nbytes, "us_per_launch": ms_k * 1e3,
                         "ring_form": {"us_per_launch": ms_ring * 1e3, "achieved": nbytes / (ms_ring * 1e-3) / 1e9,
                                       "frac": nbytes / (ms_ring * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                       "note": "append folded in: shift + decode of a linear window move 3 x these bytes"}},
            "device_status": lcm.read_status()}
    print(json.dumps(line), flush=True)


def projection_arm(args):
    """The tensor-core GEMM of the library at the training shape (8 x 16,640 rows, 768 wide): chunk K/V
    projection with the cache append as its epilogue, and its linear mode with the RMSNorm row scale
    (pre-norm + q_proj) and with the residual epilogue (o_proj + residual)."""
    import long_context_modeling_b200 as lcm
    from long_context_modeling_b200 import fused_ops as F
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    n, c, dim = 8, 260, 768
    m = n * c * 64
    g = torch.Generator(device=dev).manual_seed(5)
    xs = [torch.randn(n, c, 64, dim, generator=g, device=dev).bfloat16() for _ in range(2)]       # 2 x 204 MB: above the L2
    wk, wv, wq = ((torch.randn(dim, dim, generator=g, device=dev) / 28).bfloat16() for _ in range(3))
    res = torch.randn(m, dim, generator=g, device=dev).bfloat16()
    out = torch.empty(m, dim, dtype=torch.bfloat16, device=dev)
    x_host = xs[0].cpu().pin_memory()
    calls = [0]

    def append_step():
        calls[0] += 1
        m2 = lcm.ChunkKVManager(zero_landmark=True, capacity=c)
        m2.append_projected(xs[calls[0] % 2], wk, wv)
        return m2

    def ev(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        sampler = ClockSampler(physical_gpu_index(0))
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps, sampler.stop()

    steps, warmup = max(args.steps, 20), max(3, args.warmup)
    with torch.no_grad():
        ms, clocks = ev(append_step, steps, warmup)
        ms_lin, _ = ev(lambda: F.linear(xs[0], wq, out=out), steps, warmup)
        ms_res, _ = ev(lambda: F.linear(xs[0], wq, residual=res, out=out), steps, warmup)
        ms_rms, _ = ev(lambda: F.linear(xs[0], wq, row_scale=F.row_rms(xs[0], 1e-5), out=out), steps, warmup)

        def e2e_step():
            m2 = lcm.ChunkKVManager(zero_landmark=True, capacity=c)
            m2.append_projected(x_host.to(dev, non_blocking=True), wk, wv)
            return m2.past_lmk_embeds[:, :1].cpu()
        ms_e2e, _ = ev(e2e_step, 5, 3)
    fl = 2 * 2 * m * dim * dim
    tf = fl / (ms * 1e-3) / 1e12
    line = {"metric": "kv_projection_append_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"chunk K/V projection with cache-append epilogue: {n} x {c} chunks x 64 rows, {dim} -> 2 x {dim} "
                                   "(cache allocation inside the step)", "rows": m, "hidden": dim,
                       "cache_policy": "two input sets of 204 MB alternate (above the 126 MB L2)"},
            "clocks": clocks,
            "e2e": {"value": fl / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": n * dim * 2, "ms_per_step": ms_e2e},
            "gpu_launches": 2 * steps,
            "linear_mode": {"rows": m, "gemm_ms": ms_lin, "gemm_tflops": fl / 2 / (ms_lin * 1e-3) / 1e12,
                            "with_residual_ms": ms_res, "rmsnorm_row_scale_ms": ms_rms},
            "roofline": {"kernel": "kv_project_append_kernel", "bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops"], "peak_source": peaks["source"] + " burst dense bf16",
                         "traffic": None, "algorithmic_flops_per_launch": fl},
            "device_status": lcm.read_status()}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# Whole-model legs of the metric: the minimal DRT body with the kernels plugged in
# --------------------------------------------------------------------------------------------
def _init_dist():
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    return dist, world, rank, local, dev


def train_arm(args):
    """One DRT-16K training step (forward + backward + fused AdamW update, autocast-free: parameters,
    activations and optimizer states in bf16) of the gpt2-small-scale DRT: 12 layers (6 lower + one group of 6 upper with GCA), 2 encoder
    layers, 768 wide, 12 heads, vocabulary 50,265, 8 sequences x 16,380 tokens (260 chunks of 63 tokens
    + landmark = 16,640 positions) per GPU, uniform random token ids.  Data-parallel over ranks: the
    gradient all-reduce of DDP is part of the step at N > 1."""
    dist, world, rank, local, dev = _init_dist()
    from long_context_modeling_b200 import drt_minimal as D
    import long_context_modeling_b200 as lcm
    torch.manual_seed(0)
    cfg = D.DRTConfig()
    model = D.DRTMinimal(cfg).to(dev).bfloat16().train()
    net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local]) if world > 1 else model
    n_seq, tokens = args.n_seq, 260 * 63
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    batches = [torch.randint(0, 50257, (n_seq, tokens), generator=g, device=dev) for _ in range(2)]

    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01, fused=True)

    def step(i):
        tok = batches[i % 2]
        opt.zero_grad(set_to_none=True)
        loss = net(tok, labels=tok)
        loss.backward()
        opt.step()
        return loss

    steps, warmup = max(3, min(args.steps, 10)), max(3, min(args.warmup, 3))
    for i in range(warmup):
        step(i)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(physical_gpu_index(local))
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        loss = step(i)
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    tok_s = world * n_seq * tokens / (ms * 1e-3)
    line = {"metric": "drt16k_train_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "one training step (forward + backward + fused AdamW update) of the minimal DRT body, gpt2-small scale: 6 lower + 6 "
                                   "upper layers with GCA, 2 encoder layers, d_model 768, 12 heads, vocab 50,265, "
                                   f"{n_seq} x 16,380 tokens per GPU, chunk 63 + landmark, top-k 8, sliding window 512 + ALiBi",
                       "n_seq_per_gpu": n_seq, "tokens_per_seq": tokens, "parameters": sum(p.numel() for p in model.parameters()),
                       "cache_policy": "activations of a step (GBs) exceed the 126 MB L2; two token batches alternate",
                       "parallelism": "data-parallel over ranks (DDP gradient all-reduce inside the step at N > 1)",
                       "note": "dense projections and MLPs are torch ops (cuBLAS); the windowed ALiBi self-attention is the flash-attn "
                               "library call the reference itself makes (model/llama.py:661-683) when that library loads, else "
                               "block-banded torch SDPA; GCA, retrieval and the chunk cache are this repository's kernels"},
            "clocks": clocks, "loss": float(loss.detach()), "device_status": lcm.read_status(),
            "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 4,
                    "note": "token ids are generated on the device; the loss is read back after the timed region"},
            "gpu_launches": None, "max_memory_gb": torch.cuda.max_memory_allocated(dev) / 1e9}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def generate_arm(args):
    """Greedy generation with a long chunk cache: 32 sequences (split over the ranks), each with
    `--cache-chunks` cached chunks (16,384 = a 1M-token context; K/V 3.2 GB + 25 MB of landmarks per
    sequence), 256 new tokens.  The caches are filled with random bf16 values (with a random-init model
    their contents are noise anyway); every decoded token runs the full minimal DRT body: 6 lower layers,
    6 upper layers with one-row GCA over the 8 retrieved chunks, and at every chunk boundary the chunk
    encoder, the cache append and the landmark retrieval over all cached chunks."""
    dist, world, rank, local, dev = _init_dist()
    from long_context_modeling_b200 import drt_minimal as D
    import long_context_modeling_b200 as lcm
    torch.manual_seed(0)
    cfg = D.DRTConfig()
    model = D.DRTMinimal(cfg).to(dev).bfloat16().eval()
    n_seq = max(1, 32 // world)
    c = args.cache_chunks
    new_tokens = 256
    state = D.DecodeState(cfg)
    # K and V in a virtual-address reservation: memory is mapped behind it as the cache fills, nothing is re-copied
    state.chunks = lcm.ChunkKVManager(group_size=1, capacity=512, zero_landmark=True, max_chunks=c + 64)
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    piece = 512
    with torch.no_grad():
        for c0 in range(0, c, piece):
            m = min(piece, c - c0)
            kv = torch.empty(n_seq, m, 64, cfg.hidden_size, dtype=torch.bfloat16, device=dev)
            kk = kv.normal_(generator=g)
            state.chunks.append(kk, kv.clone().normal_(generator=g),
                                torch.empty(n_seq, m, cfg.hidden_size, dtype=torch.bfloat16, device=dev).normal_(std=0.125, generator=g))
        nl = cfg.decoder_layers[0] + sum(cfg.decoder_layers[1:])
        w = cfg.slide_window + 1
        state.self_attn = [(torch.randn(n_seq, cfg.num_attention_heads, w, cfg.head_dim, device=dev, dtype=torch.bfloat16),
                            torch.randn(n_seq, cfg.num_attention_heads, w, cfg.head_dim, device=dev, dtype=torch.bfloat16)) for _ in range(nl)]
        state.position = c * 64
        idx0 = torch.stack([torch.randperm(c, device=dev)[:cfg.chunk_topk] for _ in range(n_seq)]).int()
        state.chunks.update_current_retrieved_chunk(idx0, torch.softmax(torch.randn(n_seq, 1, cfg.chunk_topk, device=dev), -1), 0)
        tok = torch.randint(0, 50257, (n_seq,), device=dev)
        # eager steps first (warm-up, and the launch-bound figure reported beside the headline) ...
        for _ in range(8):
            tok = model.decode_step(tok, state).argmax(-1)
        torch.cuda.synchronize()
        ee0, ee1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ee0.record()
        for _ in range(24):
            tok = model.decode_step(tok, state).argmax(-1)
        ee1.record()
        torch.cuda.synchronize()
        eager_ms = ee0.elapsed_time(ee1) / 24
        # ... then the product path: token steps between chunk boundaries replayed from a CUDA graph, boundary
        # steps (chunk encoder, cache append, landmark retrieval over all cached chunks) eager
        # fused token step by default (45,500 tokens/s; the plain graphed step through the unfused modules, with eager boundary
        # steps: 15,700)
        decoder = D.GraphedDecoder(model, state, fused=not args.plain_decode)
        tok = decoder.run(tok, 40)[:, -1].contiguous()      # warm-up across one chunk boundary (not counted)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(physical_gpu_index(local))
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        produced = decoder.run(tok, new_tokens)
        e1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    tok_s = world * n_seq * new_tokens / (ms * 1e-3)
    line = {"metric": "drt_1m_ctx_decode_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": new_tokens,
            "warmup": 72, "ms_per_step": ms / new_tokens, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"greedy generation of 256 tokens, {32} sequences in total ({n_seq} per GPU), minimal DRT body at "
                                   f"gpt2-small scale, {c} cached chunks per sequence ({c * 64} positions), top-k 8",
                       "sequences_per_gpu": n_seq, "cache_chunks": c, "new_tokens": new_tokens,
                       "cache_gb_per_gpu": n_seq * c * 64 * cfg.hidden_size * 2 * 2 / 1e9,
                       "cache_memory": "K / V in a virtual-address reservation grown 2 MB page by page (outside torch's allocator: "
                                       "not part of max_memory_gb)",
                       "cache_policy": "the chunk cache (GBs per sequence) exceeds the 126 MB L2; every boundary step scans all landmarks",
                       "parallelism": "sequences split over ranks, no collective per token",
                       "note": "the 62 token steps between two chunk boundaries are replayed from a CUDA graph (captured once: it "
                               "reads the cache through the view over all mapped chunk slots and the retrieved ids through static "
                               "buffers, so later spans replay it too; a capture inside the timed region only after new pages are "
                               "mapped); at a chunk boundary the landmark position is one more replay and only the chunk encoder, the "
                               "cache append and the retrieval run eagerly (plain decode: the whole boundary step eager); token step: "
                               + ("unfused modules" if args.plain_decode else "fused (one q|k|v and one gate|up product with the norm folded in, "
                                  "cached windows kept as rings that the attention kernel updates itself)"),
                       "eager_ms_per_step": eager_ms, "graph_captures": decoder.captures},
            "clocks": clocks, "device_status": lcm.read_status(),
            "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "note": "tokens stay on the device between steps (greedy argmax on the device)"},
            "gpu_launches": None, "max_memory_gb": torch.cuda.max_memory_allocated(dev) / 1e9}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--workload", default="gca", choices=["gca", "retrieval", "decode", "triton-ref", "train16k", "generate", "window-decode", "projection"],
                    help="gca (default, the headline): GCA fwd+bwd at the DRT-16K shape; retrieval: landmark top-k over "
                         "a 16M-token cache; decode: one-row GCA for 32 sequences; train16k: one training step of the minimal "
                         "DRT body at the DRT-16K shape; generate: greedy generation with a 1M-token chunk cache")
    ap.add_argument("--triton-ref", action="store_true",
                    help="gca workload, 1 GPU: also time the reference's own Triton kernels (staged under oracle/_ref) "
                         "in a subprocess and add the result as `reference_triton_gpu`")
    ap.add_argument("--cache-chunks", type=int, default=16384,
                    help="generate workload: cached chunks per sequence (16,384 = a 1M-token context)")
    ap.add_argument("--per-head", action="store_true", help="retrieval workload: one 64-d score and top-k per head")
    ap.add_argument("--plain-decode", action="store_true", help="generate workload: graphed token steps through the unfused modules")
    ap.add_argument("--n-seq", type=int, default=N_SEQ,
                    help="sequences per GPU (default: the DRT-16K batch of 8; smaller values are for profiling captures)")
    args = ap.parse_args()
    globals()["N_SEQ"] = args.n_seq
    if args.impl == "reference":
        reference_arm(args)
    elif args.workload == "retrieval":
        retrieval_arm(args)
    elif args.workload == "decode":
        decode_arm(args)
    elif args.workload == "triton-ref":
        triton_ref_arm(args)
    elif args.workload == "train16k":
        train_arm(args)
    elif args.workload == "window-decode":
        window_decode_arm(args)
    elif args.workload == "projection":
        projection_arm(args)
    elif args.workload == "generate":
        generate_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
