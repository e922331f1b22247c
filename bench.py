#!/usr/bin/env python
"""Benchmark of the attention path: `python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload W]`.

Prints ONE JSON line (rank 0). The default workload is BASELINE config 2 as a batch: GQA decode of 8 sequences,
1 new token each, 64 query heads, 8 key heads, head 128, 32,768 cached fp16 tokens a sequence (1 GiB of K+V on each
GPU: every step's reads miss L2). A step is one pass of the decode path over the batch.

  value     KV bytes the step must read / device time, inputs resident in HBM, summed over ranks (weak scaling: every
            rank holds its own 8 sequences; there is no exchange between independent sequences)
  e2e       the same metric through the reference's own calls with HOST buffers: per sequence ns_copy_to(q, k, v rows),
            ns_q35_kv_store, ns_q35_attn_decode, ns_copy_from(out), one ns_sync a step
  roofline  HBM: algorithmic bytes a launch / CUDA-event time of the launch, against the measured copy bandwidth
  cpu_baseline / --impl reference: the CPU restatement of the reference kernel (oracle/) on the host cores

The reference's SYCL kernels cannot be built here (no oneAPI toolchain), so the reference arm times the oracle port.
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "prefill attn TFLOP/s & decode KV-read GB/s vs roofline at 1/2/4/8 B200"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


class ClockSampler:
    """SM clock and throttle reasons of one GPU, read through NVML while the timed region runs (read-only)."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _once(self):
        nv = self.nv
        try:
            self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
            r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") else \
                nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
            for bit, name in names.items():
                if r & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def start(self):
        if not self.nv:
            return
        self._once()

        def loop():
            while not self._stop.wait(0.02):
                self._once()
        self._t = threading.Thread(target=loop, daemon=True)
        self._t.start()

    def stop(self):
        if not self.nv:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self._once()
        self._stop.set()
        if self._t:
            self._t.join()
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ---- the workload -----------------------------------------------------------------------------------------------------

C2 = dict(T=1, Hq=64, Hkv=8, D=128, kv=32768, B=8)


def c2_bytes_per_seq(w):
    return 2 * w["kv"] * w["Hkv"] * w["D"] * 2          # K and V read once (the algorithmic figure)


def make_seq(config, w, seq):
    from nextsycl_b200 import workloads as W
    return W.gqa_case(config, w["T"], w["Hq"], w["Hkv"], w["D"], w["kv"], seq=seq)


def cpu_time_decode(w, seconds=6.0, seq=0):
    """The oracle's flash-numerics decode of ONE sequence of the workload on all host threads, repeated for about
    `seconds`; returns (bytes/s, threads, repeats)."""
    from oracle import oracle as O
    q, k, v, p0 = make_seq(2, w, seq)
    qf, kb, vb = q.astype(np.float32), k.view(np.uint16), v.view(np.uint16)
    O.gqa_flash_decode(qf, kb, vb, w["T"], w["Hq"], w["Hkv"], w["D"], w["kv"], p0)   # warm
    n, t0 = 0, time.perf_counter()
    while True:
        O.gqa_flash_decode(qf, kb, vb, w["T"], w["Hq"], w["Hkv"], w["D"], w["kv"], p0)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= seconds:
            break
    return c2_bytes_per_seq(w) * n / dt, O.threads(), n, dt / n


def run_reference(args):
    """--impl reference: the reference kernel's CPU restatement on the host cores; a step = one sequence of the batch
    (1/8 of the workload's step; the metric is a rate, so the sample size does not scale it)."""
    w = dict(C2)
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    q, k, v, p0 = make_seq(2, w, 0)
    qf, kb, vb = q.astype(np.float32), k.view(np.uint16), v.view(np.uint16)
    for _ in range(args.warmup):
        O.gqa_flash_decode(qf, kb, vb, w["T"], w["Hq"], w["Hkv"], w["D"], w["kv"], p0)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.gqa_flash_decode(qf, kb, vb, w["T"], w["Hq"], w["Hkv"], w["D"], w["kv"], p0)
    dt = (time.perf_counter() - t0) / args.steps
    gbs = c2_bytes_per_seq(w) / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": config_of(w, args.gpus),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": O.threads(), "kind": "port",
                         "sample": "one sequence of the batch (134,217,728 KV bytes) a step; CPU restatement of kernels/llm/qwen35/silo/attn.cpp "
                                   "decode numerics, OpenMP over (row, head); the SYCL reference itself cannot be built without oneAPI"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def config_of(w, n):
    return {"workload": "config 2: GQA decode, 1 new token, 64 query / 8 key heads, head 128, 32,768 cached fp16 tokens, batch 8 per GPU",
            "batch_per_gpu": w["B"], "kv_len": w["kv"], "q_heads": w["Hq"], "kv_heads": w["Hkv"], "head_dim": w["D"],
            "l2": "inputs larger than L2 (1 GiB of K+V per GPU per step)", "parallelism": f"sequences sharded, {n} GPU(s), no exchange"}


def run_ours(args):
    from nextsycl_b200 import DevBuf, Gpu, HostBuf, Ops
    w = dict(C2)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    gpu = Gpu(local)
    ops = Ops(gpu)
    T, Hq, Hkv, D, kv, B = w["T"], w["Hq"], w["Hkv"], w["D"], w["kv"], w["B"]

    # ---- inputs resident in HBM: B sequences with their own caches (distinct seeds per rank and sequence)
    seqs, qs, keep = [], [], []
    for b in range(B):
        q, k, v, p0 = make_seq(2, w, rank * B + b)
        qs.append(q)
        dk, dv = DevBuf.of(gpu, k), DevBuf.of(gpu, v)
        keep += [dk, dv]
        seqs.append((dk, dv, kv, p0))
    dq = DevBuf.of(gpu, np.stack(qs))
    table = ops.seq_table(seqs)
    out = DevBuf(gpu, B * T * Hq * D * 2)
    scratch = DevBuf(gpu, max(4, 4 * ops.gqa_decode_scratch(B, T, Hq, Hkv, D, kv)))

    def step():
        ops.gqa_decode(dq, Hq * D, T * Hq * D, table, B, T, Hq, Hkv, D, kv, out, scratch)

    def barrier():
        gpu.sync()
        if dist:
            import torch
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        a = gpu.stamp()
        for _ in range(steps):
            fn()
        b = gpu.stamp()
        gpu.sync()
        ms = gpu.elapsed_ns(a, b) / 1e6
        barrier()
        if dist:
            import torch
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local)
    sampler.start()
    ms = timed(step, args.steps, max(3, args.warmup))
    clocks = sampler.stop()
    ms_step = ms / args.steps
    bytes_step = B * c2_bytes_per_seq(w)
    value = world * bytes_step / (ms_step * 1e-3) / 1e9

    if args.kernel_only:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "ms_per_step": ms_step,
                              "kernel_only": True, "clocks": clocks}))
        if dist:
            dist.destroy_process_group()
        gpu.close()
        return

    # ---- end to end through the reference's calls, host buffers in, host buffer out
    hq = HostBuf(gpu, B * Hq * D * 4)
    hk = HostBuf(gpu, B * Hkv * D * 4)
    hv = HostBuf(gpu, B * Hkv * D * 4)
    ho = HostBuf(gpu, B * Hq * D * 4)
    from nextsycl_b200 import workloads as W
    hq.array(np.float32)[:] = np.stack(qs).astype(np.float32).ravel()
    hk.array(np.float32)[:] = W.rng(2, 9001 + rank).standard_normal(B * Hkv * D, dtype=np.float32)
    hv.array(np.float32)[:] = W.rng(2, 9002 + rank).standard_normal(B * Hkv * D, dtype=np.float32)
    dqf = DevBuf(gpu, B * Hq * D * 4)
    dkf = DevBuf(gpu, B * Hkv * D * 4)
    dvf = DevBuf(gpu, B * Hkv * D * 4)
    dof = DevBuf(gpu, B * Hq * D * 4)
    sc1 = DevBuf(gpu, max(4, 4 * ops.attn_decode_scratch(T, Hq, Hkv, D, kv - 1)))
    api, raw = gpu.api, gpu.raw

    views = [(dkf.view(b * Hkv * D * 4, Hkv * D * 4), dvf.view(b * Hkv * D * 4, Hkv * D * 4), dqf.view(b * Hq * D * 4, Hq * D * 4),
              dof.view(b * Hq * D * 4, Hq * D * 4)) for b in range(B)]

    def e2e_step():
        api.ns_copy_to(raw, dqf.ptr, hq.ptr, hq.len)
        api.ns_copy_to(raw, dkf.ptr, hk.ptr, hk.len)
        api.ns_copy_to(raw, dvf.ptr, hv.ptr, hv.len)
        for b in range(B):
            dk, dv, cap, p0 = seqs[b]
            kq, vq, qq, oq = views[b]
            ops.kv_store(kq, Hkv * D, vq, Hkv * D, 1, Hkv, D, cap, p0, dk, dv)
            ops.attn_decode(qq, Hq * D, dk, dv, T, Hq, Hkv, D, cap, p0, oq, sc1)
        api.ns_copy_from(raw, ho.ptr, dof.ptr, ho.len)
        gpu.sync()

    e2e_steps = max(5, min(args.steps, 200))
    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if dist:
        import torch
        t = torch.tensor([e2e_s], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_val = world * bytes_step / e2e_s / 1e9

    if rank == 0:
        pk = peaks()
        hbm = float(pk["hbm_gbs"])
        per_gpu = bytes_step / (ms_step * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": config_of(w, world),
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": hbm, "unit": "GB/s", "frac": per_gpu / hbm, "traffic": None,
                         "peak_source": pk["_source"],
                         "note": "per GPU; algorithmic bytes = 2*kv*Hkv*D*2 B a sequence x 8 sequences a launch; duration = CUDA-event time of a "
                                 "step (the split kernel plus its merge kernel)"},
            "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": int(hq.len + hk.len + hv.len), "d2h_bytes_per_step": int(ho.len),
                    "ms_per_step": e2e_s * 1e3,
                    "path": "per sequence: ns_copy_to q,k,v rows (pinned) -> ns_q35_kv_store -> ns_q35_attn_decode -> ns_copy_from out; ns_sync a step"},
            "gpu_launches": int(args.steps * 2),
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu:
            bps, cores, n, per = cpu_time_decode(w, seconds=args.cpu_seconds)
            line["cpu_baseline"] = {"value": bps / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                                    "sample": f"one sequence of the batch (134,217,728 KV bytes) x {n} repeats, {per * 1e3:.1f} ms each; "
                                              "CPU restatement of the reference decode kernel's numerics"}
        print(json.dumps(line))
    if dist:
        dist.destroy_process_group()
    gpu.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--cpu-seconds", type=float, default=6.0)
    ap.add_argument("--kernel-only", action="store_true", help="device-timed leg only (no end-to-end or CPU leg): for profiler runs")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
