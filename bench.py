#!/usr/bin/env python
"""Benchmark of the attention path.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME] [--no-others]

Prints ONE JSON line (rank 0). The headline workload (`decode_c2`) is benchmark configuration 2 as a batch: GQA decode of 8
sequences, 1 new token each, 64 query / 8 key heads of 128, 32,768 cached fp16 tokens a sequence - 1 GiB of K+V per
GPU, so every step's reads miss L2. A step is one pass of the path over the batch.

  value      KV bytes the step must read / device time, inputs resident in HBM, summed over ranks (weak scaling:
             every rank holds its own 8 sequences; independent sequences need no exchange)
  e2e        the same metric from HOST buffers through the library's C-ABI: the step's q | k | v rows up from one pinned
             buffer, ns_b200_kv_store_batch, ns_b200_gqa_decode, the outputs down, one ns_sync a step
  e2e_reference_symbols  the same through the reference's own per-sequence calls: ns_copy_to(q, k, v rows) ->
             ns_q35_kv_store -> ns_q35_attn_decode -> ns_copy_from(out) a sequence, one ns_sync a step
  roofline   algorithmic bytes (or flops) a launch / CUDA-event time, against the measured peaks
  cpu_baseline, --impl reference: the CPU restatement of the reference kernel (oracle/) on the host cores; the
             reference's SYCL kernels themselves cannot be built without a oneAPI toolchain
  others     the other benchmark configurations, each timed the same way for a few steps: 16K and 2K causal prefill
             (TFLOP/s), 128K and 256K decode, absorbed MLA decode at three context lengths, the bf16 MLA prefill chunk
             (heads sharded over the ranks)

`--workload NAME` makes another configuration the headline (used for profiler runs).
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
            while not self._stop.wait(0.005):
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


# ---- environment shared by the workloads ----------------------------------------------------------------------------------

class Env:
    def __init__(self):
        from nextsycl_b200 import Gpu, Ops
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.dist = None
        if self.world > 1:
            import torch
            import torch.distributed as dist
            torch.cuda.set_device(self.local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            self.dist = dist
            self.torch = torch
        self.gpu = Gpu(self.local)
        self.ops = Ops(self.gpu)

    def barrier(self):
        self.gpu.sync()
        if self.dist:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max_over_ranks(self, x):
        if not self.dist:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, fn, steps, warmup, sampler=None, min_ms=0.0):
        """W warm-up steps, then K steps between two stamps on the library's compute stream; barrier + sync on both
        sides; the maximum over ranks. `sampler` (a ClockSampler) runs over the timed region only. With `min_ms`, K grows
        (the same on every rank) until the timed region lasts about that long, so that the clock samples are samples under
        this load. Returns (milliseconds a step, K)."""
        for _ in range(warmup):
            fn()
        if min_ms > 0:
            self.barrier()
            a = self.gpu.stamp()
            for _ in range(3):
                fn()
            b = self.gpu.stamp()
            self.gpu.sync()
            est = self.max_over_ranks(self.gpu.elapsed_ns(a, b) / 3e6)
            steps = int(max(steps, min(20000, -(-min_ms // max(est, 1e-4)))))
        self.barrier()
        if sampler:
            sampler.start()
        a = self.gpu.stamp()
        for _ in range(steps):
            fn()
        b = self.gpu.stamp()
        self.gpu.sync()
        self.clocks = sampler.stop() if sampler else None
        ms = self.gpu.elapsed_ns(a, b) / 1e6
        self.barrier()
        return self.max_over_ranks(ms) / steps, steps

    def close(self):
        if self.dist:
            self.dist.destroy_process_group()
        self.gpu.close()


def device_random_f16(env, nbytes, seed, sigma=1.0, bf16=False):
    """A device buffer of `nbytes` of seeded N(0, sigma) 16-bit values: a 32 MiB host block drawn once and copied
    end to end (the values repeat every 16 Mi elements, which no kernel here can profit from)."""
    from nextsycl_b200 import DevBuf
    from nextsycl_b200 import workloads as W
    from nextsycl_b200.core import check
    block_elems = min(nbytes // 2, 16 << 20)
    blk = W.normal_bf16_bits(90, seed, (block_elems,), sigma) if bf16 else W.normal_f16(90, seed, (block_elems,), sigma)
    buf = DevBuf(env.gpu, nbytes)
    buf.write(blk)
    env.gpu.sync()
    done = block_elems * 2
    while done < nbytes:
        n = min(done, nbytes - done)
        check(env.gpu.api, env.gpu.api.ns_copy_dev(env.gpu.raw, buf.ptr + done, buf.ptr, n), "copy_dev")
        done += n
    env.gpu.sync()
    return buf


CALLS_A_REPLAY = 16


def replay_in_turn(env, one, rotate):
    """ONE recorded graph of at least CALLS_A_REPLAY consecutive calls, `one(r)` over the `rotate` input sets in turn.
    Returns (step, calls, graph): a step submits the graph once and stands for `calls` calls. A submission of its own per
    call puts about 2 us of the GPU's front end between two short kernels (times of single-kernel replays come out as
    multiples of 2.04 us), which an engine that replays a whole decode step - dozens of layers in one submission - never
    pays; per call inside one submission is what the kernels take."""
    calls = -(-CALLS_A_REPLAY // rotate) * rotate
    g = env.gpu.record(lambda: [one(r % rotate) for r in range(calls)])

    def step():
        g.launch()
    return step, calls, g


# ---- workloads: each returns (step_fn, info) where info has the algorithmic work a step ------------------------------------

def wl_gqa_decode(env, T, Hq, Hkv, D, kv, B, rotate=1, real_data=True, graph=False):
    """B sequences a GPU (each its own caches); `rotate` distinct cache sets used in turn so L2 cannot hold a step's reads."""
    from nextsycl_b200 import DevBuf
    from nextsycl_b200 import workloads as W
    ops = env.ops
    sets, keep, qs = [], [], []
    for r in range(rotate):
        seqs = []
        for b in range(B):
            if real_data:
                q, k, v, p0 = W.gqa_case(2, T, Hq, Hkv, D, kv, seq=env.rank * B * rotate + r * B + b)
                dk, dv = DevBuf.of(env.gpu, k), DevBuf.of(env.gpu, v)
                if r == 0:
                    qs.append(q)
            else:
                dk = device_random_f16(env, Hkv * kv * D * 2, 100 + 2 * (r * B + b))
                dv = device_random_f16(env, Hkv * kv * D * 2, 101 + 2 * (r * B + b))
                if r == 0:
                    qs.append(W.normal_f16(2, 50 + b, (T, Hq * D)))
            keep += [dk, dv]
            seqs.append((dk, dv, kv, kv - T))
        sets.append((ops.seq_table(seqs), seqs))
    dq = DevBuf.of(env.gpu, np.stack(qs))
    out = DevBuf(env.gpu, B * T * Hq * D * 2)
    scratch = DevBuf(env.gpu, max(4, 4 * ops.gqa_decode_scratch(B, T, Hq, Hkv, D, kv)))
    i = [0]

    def one(r):
        ops.gqa_decode(dq, Hq * D, T * Hq * D, sets[r][0], B, T, Hq, Hkv, D, kv, out, scratch)
    if graph:
        # the call reads its lengths from device memory, so a recorded step stays valid: replayed as one submission
        one(0)
        env.gpu.sync()
        step, calls, g = replay_in_turn(env, one, rotate)
        keep.append(g)
    else:
        calls = 1

        def step():
            one(i[0] % rotate)
            i[0] += 1
    info = {"bytes": B * 2 * kv * Hkv * D * 2, "flops": 4 * (T * (kv - T) + T * (T + 1) // 2) * Hq * D * B, "bound": "hbm", "launches": 2,
            "keep": (keep, sets, dq, out, scratch), "qs": qs, "seqs": sets[0][1], "calls": calls}
    return step, info


def wl_gqa_decode_q35(env, kt, kv=131072):
    """One decode row of the qwen35 geometry (24 query / 4 key heads of 256) over a cache of form kt (0 fp16, 1 q8_0, 2 q4_0)
    through the reference's own symbol ns_q35_attn_decode_kv; the caches are written by ns_q35_kv_store[_q] from seeded rows.
    Two cache sets used in turn; a step is a recorded graph (the call takes its position by value)."""
    from nextsycl_b200 import DevBuf
    from nextsycl_b200 import workloads as W
    from nextsycl_b200.core import check
    api, gpu = env.gpu.api, env.gpu
    T, Hq, Hkv, D = 1, 24, 4, 256
    rb = {0: 512, 1: 272, 2: 144}[kt]
    blk = 4096
    rows = [DevBuf.of(gpu, W.normal_f32(6, 10 + i, (blk, Hkv * D))) for i in range(2)]
    sets = []
    for r in range(2):
        kc, vc = DevBuf(gpu, Hkv * kv * rb), DevBuf(gpu, Hkv * kv * rb)
        for p0 in range(0, kv, blk):
            if kt == 0:
                check(api, api.ns_q35_kv_store(gpu.raw, rows[r].ptr, Hkv * D, rows[1 - r].ptr, Hkv * D, blk, Hkv, D, kv, p0, kc.ptr, vc.ptr), "kv_store")
            else:
                check(api, api.ns_q35_kv_store_q(gpu.raw, kt, rows[r].ptr, Hkv * D, rows[1 - r].ptr, Hkv * D, blk, Hkv, D, kv, p0, kc.ptr, vc.ptr), "kv_store_q")
        sets.append((kc, vc))
    q = DevBuf.of(gpu, W.normal_f32(6, 1, (T, Hq * D)))
    out = DevBuf(gpu, T * Hq * D * 4)
    scratch = DevBuf(gpu, max(4, 4 * int(api.ns_q35_attn_decode_scratch(T, Hq, Hkv, D, kv - T))))

    def one(r):
        check(api, api.ns_q35_attn_decode_kv(gpu.raw, kt, q.ptr, Hq * D, sets[r][0].ptr, sets[r][1].ptr, T, Hq, Hkv, D, kv, kv - T, out.ptr, scratch.ptr), "decode_kv")
    one(0)
    gpu.sync()
    step, calls, graphs = replay_in_turn(env, one, 2)
    info = {"bytes": 2 * kv * Hkv * rb, "bound": "hbm", "launches": 2, "keep": (rows, sets, q, out, scratch, graphs),
            "tokens_bytes_f16": 2 * kv * Hkv * 512, "calls": calls}
    return step, info


def wl_prefill(env, T, Hq, Hkv, D):
    """Causal prefill from position 0, fp16; with several ranks each takes a contiguous share of the key heads (and their
    query heads) - no exchange. With more ranks than key heads, ranks that share a key head each take a share of its
    query heads (its K and V replicated)."""
    from nextsycl_b200 import DevBuf
    w = env.world
    if w <= Hkv:
        hkv_r, hq_r = Hkv // w, Hq // w
    else:
        hkv_r, hq_r = 1, Hq // w
    # input sets used in turn so that together they hold 300 MB (q, k, v and the output of a set are touched once a step)
    set_bytes = 2 * T * hq_r * D * 2 + 2 * hkv_r * T * D * 2
    rotate = max(2, -(-300_000_000 // set_bytes))
    sets = [(device_random_f16(env, T * hq_r * D * 2, 1 + 3 * r), device_random_f16(env, hkv_r * T * D * 2, 2 + 3 * r),
             device_random_f16(env, hkv_r * T * D * 2, 3 + 3 * r), DevBuf(env.gpu, T * hq_r * D * 2)) for r in range(rotate)]
    i = [0]

    def one(r):
        q, k, v, out = sets[r]
        env.ops.gqa_prefill(0, q, hq_r * D, k, v, T, hq_r, hkv_r, D, T, 0, out)
    keys = T * (T + 1) // 2
    calls, g = 1, None
    if 4 * keys * hq_r * D < 2e11:      # a prompt of tens of microseconds: many calls a submission, as in replay_in_turn
        one(0)
        env.gpu.sync()
        step, calls, g = replay_in_turn(env, one, rotate)
    else:
        def step():
            one(i[0] % rotate)
            i[0] += 1
    info = {"flops": 4 * keys * hq_r * D, "flops_total": 4 * keys * Hq * D, "bytes": 2 * T * hkv_r * D * 2, "bound": "tensor", "launches": 1,
            "calls": calls, "keep": (sets, g)}
    return step, info


def wl_mla_decode(env, n):
    from nextsycl_b200 import DevBuf
    from nextsycl_b200 import workloads as W
    q = DevBuf.of(env.gpu, W.normal_f16(3, 0, (1, 128, 576)))
    # as many cache sets, used in turn, as hold 300 MB together: between two uses of a set more than twice the 126 MB L2 has gone by
    rotate = max(2, -(-300_000_000 // (n * 1152)))
    whole = device_random_f16(env, rotate * n * 1152, 10, 0.5)
    caches = [whole.view(r * n * 1152, n * 1152) for r in range(rotate)]
    out = DevBuf(env.gpu, 128 * 512 * 4)
    sc = DevBuf(env.gpu, max(4, 4 * env.ops.mla_decode_scratch(1, 128, n - 1)))
    i = [0]

    def one(r):
        env.ops.mla_decode(q, caches[r], 1, 128, n - 1, float(1 / np.sqrt(192.0)), out, sc)
    one(0)
    env.gpu.sync()
    step, calls, graphs = replay_in_turn(env, one, rotate)
    info = {"bytes": 1152 * n, "flops": 278528 * n, "bound": "hbm+tensor", "launches": 2, "calls": calls, "keep": (q, whole, caches, out, sc, graphs)}
    return step, info


def wl_glm_sel_decode(env, n=131072, H=64, K=512):
    """The one attention kernel the reference publishes a time for (TODO.md:546-551: GLM-5.3's absorbed-MLA decode attention at
    128K context, 2,051 selected cells x 64 heads x 512-wide fp16 latents, 1,047 -> 444 us a layer on Arc Pro B70 / B65): one
    decode row over the indexer's 512 selected pools of 4 tokens plus the 3 tokens of its incomplete pool, through the
    reference's own symbol ns_mla_attend_sel. Cache sets in turn; the selection differs per set."""
    from nextsycl_b200 import DevBuf
    from nextsycl_b200 import workloads as W
    from nextsycl_b200.core import check
    api, gpu = env.gpu.api, env.gpu
    pos0 = n + 2                                   # (pos0 + 1) % 4 == 3: three tokens in the row's incomplete pool
    cells = pos0 + 1
    q = DevBuf.of(gpu, W.normal_f32(3, 60, (1, H * 512)))
    rotate = max(2, -(-300_000_000 // (cells * 1024)))
    whole = device_random_f16(env, rotate * cells * 1024, 61, 0.5)
    caches = [whole.view(r * cells * 1024, cells * 1024) for r in range(rotate)]
    sels = [DevBuf.of(gpu, np.sort(W.rng(3, 62 + r).choice((pos0 + 1) // 4, size=K, replace=False)).astype(np.int32)) for r in range(rotate)]
    cnt = DevBuf.of(gpu, np.array([K], np.int32))
    out = DevBuf(gpu, H * 512 * 4)

    def one(r):
        check(api, api.ns_mla_attend_sel(gpu.raw, q.ptr, caches[r].ptr, out.ptr, 1, H, 512, pos0, np.float32(1 / 16.0), sels[r].ptr, cnt.ptr, K), "ns_mla_attend_sel")
    one(0)
    gpu.sync()
    step, calls, graphs = replay_in_turn(env, one, rotate)
    info = {"bytes": (4 * K + 3) * 1024, "flops": (4 * K + 3) * H * 2 * (512 + 512), "bound": "hbm", "launches": 3, "calls": calls,
            "keep": (q, whole, caches, sels, cnt, out, graphs),
            "published": {"reference_us": 444.0, "reference_us_before": 1047.0, "hardware": "Intel Arc Pro B70 / B65 (608 GB/s)",
                          "source": "TODO.md:546-551 (per layer and pass, 2,051 cells x 64 heads, fp16 latents)"}}
    return step, info


def wl_ds2_decode(env, n):
    """The reference's whole deepseek2 decode op for one row (ns_ds2_mla_decode: absorb q through k_b, the latent attention of
    config 3, out through v_b), fp32 rows in and out, 128 heads; cache sets in turn as in wl_mla_decode."""
    from nextsycl_b200 import DevBuf
    from nextsycl_b200 import workloads as W
    from nextsycl_b200.core import check
    api, gpu = env.gpu.api, env.gpu
    H = 128
    q = DevBuf.of(gpu, W.normal_f32(3, 40, (1, H * 192)))
    kb = DevBuf.of(gpu, W.normal_f16(3, 41, (H, 512, 128), 0.09))
    vb = DevBuf.of(gpu, W.normal_f16(3, 42, (H, 128, 512), 0.05))
    rotate = max(2, -(-300_000_000 // (n * 1152)))
    whole = device_random_f16(env, rotate * n * 1152, 43, 0.5)
    caches = [whole.view(r * n * 1152, n * 1152) for r in range(rotate)]
    out = DevBuf(gpu, H * 128 * 4)

    def one(r):
        check(api, api.ns_ds2_mla_decode(gpu.raw, q.ptr, kb.ptr, vb.ptr, caches[r].ptr, out.ptr, 1, H, n - 1, np.float32(1 / np.sqrt(192.0))), "ns_ds2_mla_decode")
    one(0)
    gpu.sync()
    step, calls, graphs = replay_in_turn(env, one, rotate)
    info = {"bytes": 1152 * n + 2 * H * 512 * 128 * 2, "flops": 278528 * n + 4 * H * 512 * 128, "bound": "hbm+tensor", "launches": 4, "calls": calls,
            "keep": (q, kb, vb, whole, caches, out, graphs)}
    return step, info


def wl_glm_prompt_gemms(env, tr=32, H=64, nc=2112, L=512):
    """The two batched fp16 GEMMs of the glm5next engine's prompt path for one block of 32 rows at its largest cell count
    (llm/glm5next/src/engine.rs:1925,1930): scores [64 x 2,112] = q~ . G^T and latents [64 x 512] = P . G per row, through
    the reference's own symbol ns_gemm_batch_h. Input sets in turn as elsewhere."""
    from nextsycl_b200 import DevBuf
    from nextsycl_b200.core import check
    api, raw = env.gpu.api, env.gpu.raw
    set_bytes = tr * (nc * L * 2 + H * L * 2 + H * nc * 2 + H * nc * 4 + H * L * 4)
    rotate = max(2, -(-300_000_000 // set_bytes))
    sets = [(device_random_f16(env, tr * nc * L * 2, 400 + 3 * r, 0.5), device_random_f16(env, tr * H * L * 2, 401 + 3 * r),
             device_random_f16(env, tr * H * nc * 2, 402 + 3 * r, 0.02), DevBuf(env.gpu, tr * H * nc * 4), DevBuf(env.gpu, tr * H * L * 4)) for r in range(rotate)]
    i = [0]

    def one(r):
        gh, qh, ph, sb, u = sets[r]
        check(api, api.ns_gemm_batch_h(raw, tr, 1, H, nc, L, qh.ptr, L, H * L, gh.ptr, L, nc * L, sb.ptr, nc, H * nc, 0), "scores")
        check(api, api.ns_gemm_batch_h(raw, tr, 0, H, L, nc, ph.ptr, nc, H * nc, gh.ptr, L, nc * L, u.ptr, L, H * L, 0), "values")
    one(0)
    env.gpu.sync()
    step, calls, graphs = replay_in_turn(env, one, rotate)
    info = {"flops": 2 * 2 * tr * H * nc * L, "bytes": set_bytes, "bound": "tensor", "launches": 2, "calls": calls, "keep": (sets, graphs)}
    return step, info


def wl_mla_prefill(env, T=4096, p0=32768, H=128):
    """benchmark configuration 4: 4,096 new rows over a 32,768-token cache, bf16, 192-wide keys / 128-wide values; the 128 heads
    sharded over the ranks (each rank its own heads' K and V; no exchange)."""
    from nextsycl_b200 import DevBuf
    h = H // env.world
    n = p0 + T
    q = device_random_f16(env, T * h * 192 * 2, 20, bf16=True)
    k = device_random_f16(env, n * h * 192 * 2, 21, bf16=True)
    v = device_random_f16(env, n * h * 128 * 2, 22, bf16=True)
    out = DevBuf(env.gpu, T * h * 128 * 2)

    def step():
        env.ops.mla_prefill(q, h * 192, k, h * 192, v, h * 128, T, h, p0, float(1 / np.sqrt(192.0)), out)
    keys = T * p0 + T * (T + 1) // 2
    info = {"flops": keys * h * 2 * (192 + 128), "flops_total": keys * H * 2 * (192 + 128), "bytes": n * h * (192 + 128) * 2, "bound": "tensor",
            "launches": 1, "keep": (q, k, v, out)}
    return step, info


def wl_kvsplit_decode(env, T=4, Hq=32, Hkv=4, D=128, kv=262144, mode="fused"):
    """benchmark configuration 5 over the ranks: each rank holds kv/N keys of every key head; a step is this rank's split-KV
    decode, the push of its partial into every rank's mailbox over NVLink, and the combine of what arrived in its own
    (strong scaling: the context is fixed, the ranks share it). mode "fused": the step as ONE kernel (ns_b200_kvsplit_step);
    "launches": the same protocol as three dependent launches (ns_b200_kvsplit_decode + _combine); "nccl": the exchange as a
    library all-gather (ns_b200_kvsplit_partial -> torch.distributed.all_gather_into_tensor over NCCL on the library's stream ->
    ns_b200_kvsplit_merge), launched from the host every step - the baseline the other two are measured against."""
    from nextsycl_b200 import DevBuf
    from nextsycl_b200 import workloads as W
    from nextsycl_b200.dist import KvSplit, key_ranges
    base, count = key_ranges(kv, env.world)[env.rank]
    assert count > 0, "a context shorter than the ranks' shares is not a benchmark case"

    def exchange(h):
        got = [None] * env.world
        env.dist.all_gather_object(got, h)
        return got
    if env.world == 1:
        box = DevBuf(env.gpu, KvSplit.mailbox_bytes(env.gpu.api, 1, T, Hq, D))
        box.fill(0)
        grp = KvSplit(env.gpu, 0, 1, T, Hq, D, local_mailboxes=[box])
    else:
        grp = KvSplit(env.gpu, env.rank, env.world, T, Hq, D, exchange=exchange)
    q = DevBuf.of(env.gpu, W.normal_f16(5, 0, (T, Hq * D)))
    rotate = 2 if count * Hkv * D * 4 > 100e6 else 4
    caches = [(device_random_f16(env, Hkv * count * D * 2, 200 + 2 * r + 16 * env.rank), device_random_f16(env, Hkv * count * D * 2, 201 + 2 * r + 16 * env.rank))
              for r in range(rotate)]
    sc = DevBuf(env.gpu, 4 * grp.scratch_floats(Hkv, count))
    out = DevBuf(env.gpu, T * Hq * D * 2)
    env.barrier()

    nccl = None
    if mode == "nccl":
        import torch
        api, raw = env.gpu.api, env.gpu.raw
        rows = T * Hq
        if env.dist:
            stream = torch.cuda.ExternalStream(env.gpu.stream(), device=torch.device("cuda", env.local))
            t_part = torch.empty(rows * (D + 2), dtype=torch.float32, device="cuda")
            t_all = torch.empty(env.world * rows * (D + 2), dtype=torch.float32, device="cuda")
            part_ptr, all_ptr = t_part.data_ptr(), t_all.data_ptr()
            nccl = (torch, stream, t_part, t_all)
        else:
            both = DevBuf(env.gpu, rows * (D + 2) * 4)
            part_ptr = all_ptr = both.ptr
            nccl = (None, None, both, both)

    def one(r):
        kc, vc = caches[r]
        if mode == "fused":
            grp.step(q, Hq * D, kc, vc, Hkv, count, base, kv - T, sc, out, epoch=0, wait_us=500000)   # step numbers kept on the device
        elif mode == "launches":
            grp.decode(q, Hq * D, kc, vc, Hkv, count, base, kv - T, sc, epoch=0)
            grp.combine(out, epoch=0, wait_us=500000)
        else:
            from nextsycl_b200.core import check
            check(api, api.ns_b200_kvsplit_partial(raw, q.ptr, Hq * D, kc.ptr, vc.ptr, T, Hq, Hkv, D, count, base, kv - T, sc.ptr, part_ptr), "partial")
            if nccl[0] is not None:
                with nccl[0].cuda.stream(nccl[1]):
                    env.dist.all_gather_into_tensor(nccl[3], nccl[2])
            check(api, api.ns_b200_kvsplit_merge(raw, all_ptr, env.world, T, Hq, D, out.ptr), "merge")
    one(0)
    env.barrier()
    i = [0]
    if mode == "nccl":
        def step():
            one(i[0] % rotate)
            i[0] += 1
        graphs = None
    else:
        # a step is recorded once per cache set and replayed: one submission, so the ranks' hosts do not set the pace
        graphs = [env.gpu.record(lambda r=r: one(r)) for r in range(rotate)]

        def step():
            graphs[i[0] % rotate].launch()
            i[0] += 1
    def check():
        """After the timed region: one more step on cache set 0; every rank's rows must be the same bits, and rank 0 holds
        them to the CPU checker's decode of the WHOLE context, rebuilt on the host from the ranks' seeds (a combine that
        merged the wrong buffer, or a rank that pushed stale partials, shows here, not in the timing)."""
        one(0)
        env.gpu.sync()
        mine = out.read(np.float16).reshape(T, Hq * D)
        rows = [mine.tobytes()]
        if env.dist:
            rows = [None] * env.world
            env.dist.all_gather_object(rows, mine.tobytes())
        same = all(r == rows[0] for r in rows)
        res = {"ranks_bit_equal": bool(same)}
        if env.rank == 0:
            from oracle import oracle as O
            O.use_all_cores()
            K = np.empty((Hkv, kv, D), np.float16)
            V = np.empty((Hkv, kv, D), np.float16)
            for r, (b, c) in enumerate(key_ranges(kv, env.world)):
                if c == 0:
                    continue
                n = Hkv * c * D
                for dst, seed in ((K, 200 + 16 * r), (V, 201 + 16 * r)):
                    blk = W.normal_f16(90, seed, (min(n, 16 << 20),))
                    dst[:, b:b + c] = np.resize(blk, n).reshape(Hkv, c, D)    # the device buffer is that block end to end
            qh = W.normal_f16(5, 0, (T, Hq * D))
            want = O.gqa_flash_decode(qh.astype(np.float32), K.view(np.uint16), V.view(np.uint16), T, Hq, Hkv, D, kv, kv - T)
            d = np.abs(mine.astype(np.float32) - want)
            res.update({"max_abs": float(d.max()), "ok": bool(same and np.all(d <= 2e-3 + 1e-2 * np.abs(want))),
                        "against": "CPU checker (flash numerics) over all %d keys; tolerance 2e-3 + 1e-2 |want|" % kv})
        return res
    info = {"bytes": 2 * count * Hkv * D * 2, "bytes_total": 2 * kv * Hkv * D * 2, "flops": 0, "bound": "hbm", "launches": 1 if mode == "fused" else 3,
            "keep": (grp, q, caches, sc, out, graphs, nccl), "check": check}
    return step, info


def wl_mla_kvsplit(env, n=131072, H=128):
    """benchmark configuration 3 at 131,072 cells with the latent cache split over the ranks by cell ranges: this rank's cells on
    the tensor cores, its partial pushed into every rank's mailbox over NVLink, the combine of what arrived in its own."""
    from nextsycl_b200 import DevBuf
    from nextsycl_b200 import workloads as W
    from nextsycl_b200.dist import KvSplit, key_ranges
    T = 1
    scale = float(1 / np.sqrt(192.0))
    base, count = key_ranges(n, env.world)[env.rank]

    def exchange(h):
        got = [None] * env.world
        env.dist.all_gather_object(got, h)
        return got
    if env.world == 1:
        box = DevBuf(env.gpu, KvSplit.mailbox_bytes(env.gpu.api, 1, T, H, 512))
        box.fill(0)
        grp = KvSplit(env.gpu, 0, 1, T, H, 512, local_mailboxes=[box])
    else:
        grp = KvSplit(env.gpu, env.rank, env.world, T, H, 512, exchange=exchange)
    q = DevBuf.of(env.gpu, W.normal_f16(3, 0, (T, H, 576)))
    rotate = max(2, -(-300_000_000 // (count * 1152)))
    whole = device_random_f16(env, rotate * count * 1152, 300 + env.rank, 0.5)
    caches = [whole.view(r * count * 1152, count * 1152) for r in range(rotate)]
    sc = DevBuf(env.gpu, 4 * grp.mla_scratch_floats(count))
    out = DevBuf(env.gpu, T * H * 512 * 4)
    env.barrier()

    def one(r):
        grp.mla_decode(q, caches[r], count, base, n - T, scale, sc, epoch=0)
        grp.mla_combine(out, epoch=0, wait_us=500000)
    one(0)
    env.barrier()
    graphs = [env.gpu.record(lambda r=r: one(r)) for r in range(rotate)]
    i = [0]

    def step():
        graphs[i[0] % rotate].launch()
        i[0] += 1

    def check():
        """One more step on cache set 0: every rank's rows the same bits; rank 0 holds 16 heads spread over the tile to the CPU
        checker's decode of the WHOLE cache, rebuilt on the host from the ranks' seeds."""
        one(0)
        env.gpu.sync()
        mine = out.read(np.float32).reshape(T, H, 512)
        rows = [mine.tobytes()]
        if env.dist:
            rows = [None] * env.world
            env.dist.all_gather_object(rows, mine.tobytes())
        res = {"ranks_bit_equal": bool(all(r == rows[0] for r in rows))}
        if env.rank == 0:
            from oracle import oracle as O
            O.use_all_cores()
            cache = np.empty((n, 576), np.float16)
            for r, (b, c) in enumerate(key_ranges(n, env.world)):
                tot = max(2, -(-300_000_000 // (c * 1152))) * c * 576
                blk = W.normal_f16(90, 300 + r, (min(tot, 16 << 20),), 0.5)
                cache[b:b + c] = np.resize(blk, c * 576).reshape(c, 576)     # cache set 0 = the buffer's first c cells
            heads = [0, 31, 32, 63, 64, 95, 96, 127, 7, 16, 45, 50, 77, 88, 101, 120]
            qh = W.normal_f16(3, 0, (T, H, 576))
            want = O.mla_gemm(np.ascontiguousarray(qh[:, heads].astype(np.float32)), cache.view(np.uint16), T, len(heads), 512, 64, n - T, np.float32(scale))
            d = np.abs(mine[:, heads] - want)
            res.update({"max_abs": float(d.max()), "ok": bool(res["ranks_bit_equal"] and np.all(d <= 2e-3 + 1e-2 * np.abs(want))),
                        "against": "CPU checker (GEMM-form numerics) over all %d cells, 16 of the 128 heads; tolerance 2e-3 + 1e-2 |want|" % n})
        return res
    info = {"bytes": 1152 * count, "bytes_total": 1152 * n, "flops": 278528 * count, "bound": "hbm", "launches": 3,
            "keep": (grp, q, whole, caches, sc, out, graphs), "check": check}
    return step, info


def measure(env, name, steps, warmup, min_ms=0.0):
    """Builds the workload, times it under a clock sampler, returns a result dict (per GPU figures plus the whole-job rate)."""
    pk = peaks()
    if name == "decode_c2":
        step, info = wl_gqa_decode(env, 1, 64, 8, 128, 32768, 8)
    elif name == "decode_c2_b1":
        step, info = wl_gqa_decode(env, 1, 64, 8, 128, 32768, 1, rotate=3, graph=True)
    elif name == "decode_128k":
        step, info = wl_gqa_decode(env, 1, 64, 8, 128, 131072, 1, rotate=2, real_data=False, graph=True)
    elif name == "decode_c5":
        step, info = wl_gqa_decode(env, 4, 32, 4, 128, 262144, 1, rotate=2, real_data=False, graph=True)
    elif name == "decode_c5_split":
        step, info = wl_kvsplit_decode(env)
    elif name == "decode_c5_split_3launch":
        step, info = wl_kvsplit_decode(env, mode="launches")
    elif name == "decode_c5_split_nccl":
        step, info = wl_kvsplit_decode(env, mode="nccl")
    elif name.startswith("decode_split_kv"):      # decode_split_kv<tokens>: the same with another context length
        step, info = wl_kvsplit_decode(env, kv=int(name[len("decode_split_kv"):]))
    elif name.startswith("decode_q35_"):
        step, info = wl_gqa_decode_q35(env, {"f16": 0, "q8": 1, "q4": 2}[name.split("_")[-1]])
    elif name == "prefill_16k":
        step, info = wl_prefill(env, 16384, 16, 4, 128)
    elif name == "prefill_c1":
        step, info = wl_prefill(env, 2048, 16, 4, 128)
    elif name == "prefill_q35_16k":
        step, info = wl_prefill(env, 16384, 24, 4, 256)
    elif name == "ds2_decode_32k":
        step, info = wl_ds2_decode(env, 32768)
    elif name == "glm_sel_decode_2051":
        step, info = wl_glm_sel_decode(env)
    elif name == "mla_decode_131k_split":
        step, info = wl_mla_kvsplit(env)
    elif name.startswith("mla_decode_"):
        step, info = wl_mla_decode(env, {"4k": 4096, "32k": 32768, "131k": 131072}[name.split("_")[-1]])
    elif name == "mla_prefill_c4":
        step, info = wl_mla_prefill(env)
    elif name == "mla_prefill_c4_h16":      # one rank's share of config 4 at 8 GPUs (16 of the 128 heads): the profiler's case
        step, info = wl_mla_prefill(env, H=16 * env.world)
    elif name == "glm_prompt_gemms":
        step, info = wl_glm_prompt_gemms(env)
    else:
        raise SystemExit(f"unknown workload {name}")
    ms, steps = env.timed(step, steps, max(3, warmup), sampler=ClockSampler(env.local), min_ms=min_ms)
    calls = info.get("calls", 1)      # calls a timed submission (replay_in_turn): the figures below are per call
    ms, steps = ms / calls, steps * calls
    res = {"workload": name, "ms_per_step": ms, "steps": steps, "clocks": env.clocks}
    if calls > 1:
        res["calls_a_submission"] = calls
    if env.clocks and env.clocks.get("sm_mhz"):
        res["ms_x_mhz"] = ms * env.clocks["sm_mhz"]
    if "tensor" in info["bound"]:
        tf = info["flops"] / (ms * 1e-3) / 1e12
        res.update({"tflops_per_gpu": tf, "frac_of_bf16_peak": tf / float(pk["bf16_tflops"]),
                    "frac_of_bf16_sustained": tf / float(pk.get("bf16_tflops_sustained", pk["bf16_tflops"]))})
        if "flops_total" in info:
            res["tflops_job"] = info["flops_total"] / (ms * 1e-3) / 1e12
    if "hbm" in info["bound"]:
        gbs = info["bytes"] / (ms * 1e-3) / 1e9
        res.update({"gbs_per_gpu": gbs, "frac_of_hbm_peak": gbs / float(pk["hbm_gbs"])})
        if "bytes_total" in info:
            res["gbs_job"] = info["bytes_total"] / (ms * 1e-3) / 1e9
        if "tokens_bytes_f16" in info:   # a quantised cache: the same tokens as so many fp16 bytes a second
            res["f16_equivalent_gbs"] = info["tokens_bytes_f16"] / (ms * 1e-3) / 1e9
    if "published" in info:   # the reference's own published time for this kernel (other hardware): ours beside it
        res["published"] = dict(info["published"], ours_us=ms * 1e3, ratio=info["published"]["reference_us"] / (ms * 1e3))
    res["_info"] = info
    return res


# dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernel, per launch and GPU, from the ncu captures summarised under
# profiles/ (a profiler's figure, constant for a workload; not measured by this script)
NCU_TRAFFIC = {"decode_c2": 1.073912e9 + 12.0e6, "mla_decode_32k": 37.96e6 + 0.07e6, "decode_q35_q8": 285.29e6 + 3.9e6}

OTHERS_1GPU = [("prefill_16k", 10), ("prefill_c1", 50), ("prefill_q35_16k", 10), ("decode_c2_b1", 50), ("decode_128k", 30), ("decode_c5", 30), ("decode_q35_f16", 30),
               ("decode_q35_q8", 30), ("decode_q35_q4", 30), ("mla_decode_4k", 50),
               ("mla_decode_32k", 50), ("mla_decode_131k", 30), ("ds2_decode_32k", 50), ("glm_sel_decode_2051", 50), ("glm_prompt_gemms", 50), ("mla_prefill_c4", 10)]
OTHERS_NGPU = [("decode_c5_split", 50), ("decode_c5_split_3launch", 50), ("decode_c5_split_nccl", 50), ("mla_decode_131k_split", 50), ("prefill_16k", 10), ("mla_prefill_c4", 10)]


def config_of(name, n):
    texts = {
        "decode_c2": "config 2: GQA decode, 1 new token, 64 query / 8 key heads, head 128, 32,768 cached fp16 tokens, batch 8 per GPU",
        "prefill_16k": "16K causal GQA prefill, 16 query / 4 key heads of 128, fp16 (config 1's geometry at the target length)",
        "prefill_c1": "config 1: causal GQA prefill, 2,048 rows, 16 query / 4 key heads of 128, fp16",
        "prefill_q35_16k": "16K causal GQA prefill of the qwen35 geometry, 24 query / 4 key heads of 256, fp16",
        "decode_c2_b1": "config 2, one sequence",
        "decode_128k": "128K GQA decode, 64 query / 8 key heads of 128, one sequence (512 MiB of K+V)",
        "decode_c5": "config 5 on one GPU: 4 verify rows, 32 query / 4 key heads of 128, 262,144 cached tokens (512 MiB of K+V)",
        "decode_q35_f16": "qwen35 geometry: 1 decode row, 24 query / 4 key heads of 256, 131,072 cached tokens, fp16 caches (ns_q35_attn_decode_kv)",
        "decode_q35_q8": "the same over q8_0 caches (272-byte rows)",
        "decode_q35_q4": "the same over q4_0 caches (144-byte rows)",
        "decode_c5_split": "config 5 over the ranks: 262,144 cached tokens split by key ranges, partials pushed over NVLink and combined, the step one kernel (strong scaling)",
        "decode_c5_split_3launch": "the same protocol as three dependent launches (split decode, merge + push, combine)",
        "decode_c5_split_nccl": "the same split with the partials exchanged by an NCCL all-gather launched from the host every step (baseline)",
        "mla_decode_131k_split": "config 3 at 131,072 cells, the latent cache split by cell ranges over the ranks, partials pushed over NVLink and combined (strong scaling)",
        "ds2_decode_32k": "ns_ds2_mla_decode, the reference's whole decode op around config 3's attention: fp32 q [128 x 192] absorbed through k_b, 32,768 cells, out through v_b",
        "mla_decode_4k": "config 3: absorbed MLA decode, 128 heads, 576-wide latent cache, 4,096 cells",
        "mla_decode_32k": "config 3, 32,768 cells",
        "mla_decode_131k": "config 3, 131,072 cells",
        "glm_sel_decode_2051": "ns_mla_attend_sel: glm5next decode attention at 128K context, 2,051 selected cells x 64 heads x 512 (the one attention kernel the reference publishes a time for)",
        "glm_prompt_gemms": "ns_gemm_batch_h twice: the glm5next prompt path's scores and latents GEMMs for 32 rows x 64 heads over 2,112 gathered cells of 512",
        "mla_prefill_c4": "config 4: bf16 MLA prefill chunk, 4,096 rows over 32,768 cached, 128 heads (192/128), heads sharded over ranks",
    }
    return {"workload": texts.get(name, name), "name": name,
            "l2": "inputs larger than L2, or several input sets used in turn",
            "submissions": "a workload whose entry carries calls_a_submission is timed as replays of ONE recorded graph of that many "
                           "consecutive calls (the input sets in turn) and reported per call; the rest one call a submission",
            "parallelism": f"{n} GPU(s)"}


# ---- reference arm --------------------------------------------------------------------------------------------------------

def cpu_decode_rate(seconds, steps=None, warmup=1):
    """The oracle's flash-numerics decode of ONE sequence of config 2 on all host threads; (bytes/s, threads, repeats, s each)."""
    from nextsycl_b200 import workloads as W
    from oracle import oracle as O
    O.use_all_cores()   # a process launcher may have exported OMP_NUM_THREADS=1: the CPU arm is an all-core figure at every N
    T, Hq, Hkv, D, kv = 1, 64, 8, 128, 32768
    q, k, v, p0 = W.gqa_case(2, T, Hq, Hkv, D, kv, seq=0)
    qf, kb, vb = q.astype(np.float32), k.view(np.uint16), v.view(np.uint16)
    for _ in range(warmup):
        O.gqa_flash_decode(qf, kb, vb, T, Hq, Hkv, D, kv, p0)
    n, t0 = 0, time.perf_counter()
    while True:
        O.gqa_flash_decode(qf, kb, vb, T, Hq, Hkv, D, kv, p0)
        n += 1
        dt = time.perf_counter() - t0
        if (steps is not None and n >= steps) or (steps is None and dt >= seconds):
            break
    return 2 * kv * Hkv * D * 2 * n / dt, O.threads(), n, dt / n


def run_reference(args):
    """--impl reference: the reference kernel's CPU restatement on the host cores. A step is one sequence of the batch
    (1/8 of the headline step); the metric is a rate, so the sample size does not scale it."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    bps, cores, n, per = cpu_decode_rate(0, steps=max(1, args.steps), warmup=max(1, args.warmup))
    gbs = bps / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": dict(config_of("decode_c2", args.gpus), sample="one sequence of the batch a step (a rate: the sample size does not scale it)"),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": "one sequence of the batch (134,217,728 KV bytes) a step; CPU restatement of the decode numerics of "
                                   "kernels/llm/qwen35/silo/attn.cpp, OpenMP over (row, head); the SYCL reference cannot be built without oneAPI"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---- our arm --------------------------------------------------------------------------------------------------------------

def e2e_decode(env, info, steps):
    """Config 2 through the reference's own calls from pinned host buffers; seconds a step (max over ranks)."""
    from nextsycl_b200 import DevBuf, HostBuf
    from nextsycl_b200 import workloads as W
    gpu, ops = env.gpu, env.ops
    T, Hq, Hkv, D, kv, B = 1, 64, 8, 128, 32768, 8
    seqs, qs = info["seqs"], info["qs"]
    hq, hk, hv, ho = HostBuf(gpu, B * Hq * D * 4), HostBuf(gpu, B * Hkv * D * 4), HostBuf(gpu, B * Hkv * D * 4), HostBuf(gpu, B * Hq * D * 4)
    hq.array(np.float32)[:] = np.stack(qs).astype(np.float32).ravel()
    hk.array(np.float32)[:] = W.rng(2, 9001 + env.rank).standard_normal(B * Hkv * D, dtype=np.float32)
    hv.array(np.float32)[:] = W.rng(2, 9002 + env.rank).standard_normal(B * Hkv * D, dtype=np.float32)
    dqf, dkf, dvf, dof = DevBuf(gpu, hq.len), DevBuf(gpu, hk.len), DevBuf(gpu, hv.len), DevBuf(gpu, ho.len)
    sc1 = DevBuf(gpu, max(4, 4 * ops.attn_decode_scratch(T, Hq, Hkv, D, kv - 1)))
    api, raw = gpu.api, gpu.raw
    views = [(dkf.view(b * Hkv * D * 4, Hkv * D * 4), dvf.view(b * Hkv * D * 4, Hkv * D * 4), dqf.view(b * Hq * D * 4, Hq * D * 4),
              dof.view(b * Hq * D * 4, Hq * D * 4)) for b in range(B)]

    def step():
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

    for _ in range(3):
        step()
    env.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    s = (time.perf_counter() - t0) / steps
    return env.max_over_ranks(s), int(hq.len + hk.len + hv.len), int(ho.len)


def e2e_decode_native(env, info, steps):
    """Config 2 from pinned host buffers through the native batched calls: ONE copy up (the step's queries as fp16 and the new
    K and V rows as fp32, packed in one pinned buffer), ONE ns_b200_kv_store_batch, ONE ns_b200_gqa_decode, ONE copy down (the
    outputs, fp16), one sync."""
    from nextsycl_b200 import DevBuf, HostBuf
    from nextsycl_b200 import workloads as W
    gpu, ops = env.gpu, env.ops
    T, Hq, Hkv, D, kv, B = 1, 64, 8, 128, 32768, 8
    seqs, qs = info["seqs"], info["qs"]
    qb, kb = B * Hq * D * 2, B * Hkv * D * 4
    hin, ho = HostBuf(gpu, qb + 2 * kb), HostBuf(gpu, B * Hq * D * 2)
    hin.array(np.float16, at=0, shape=(B * Hq * D,))[:] = np.stack(qs).ravel()
    hin.array(np.float32, at=qb, shape=(B * Hkv * D,))[:] = W.rng(2, 9001 + env.rank).standard_normal(B * Hkv * D, dtype=np.float32)
    hin.array(np.float32, at=qb + kb, shape=(B * Hkv * D,))[:] = W.rng(2, 9002 + env.rank).standard_normal(B * Hkv * D, dtype=np.float32)
    din, do = DevBuf(gpu, hin.len), DevBuf(gpu, ho.len)
    dq, dkf, dvf = din.view(0, qb), din.view(qb, kb), din.view(qb + kb, kb)
    table = ops.seq_table(seqs)
    sc = DevBuf(gpu, max(4, 4 * ops.gqa_decode_scratch(B, T, Hq, Hkv, D, kv)))
    api, raw = gpu.api, gpu.raw

    def step():
        api.ns_copy_to(raw, din.ptr, hin.ptr, hin.len)
        ops.kv_store_batch(dkf, Hkv * D, T * Hkv * D, dvf, Hkv * D, T * Hkv * D, table, B, T, Hkv, D)
        ops.gqa_decode(dq, Hq * D, T * Hq * D, table, B, T, Hq, Hkv, D, kv, do, sc)
        api.ns_copy_from(raw, ho.ptr, do.ptr, ho.len)
        gpu.sync()

    for _ in range(3):
        step()
    env.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    s = (time.perf_counter() - t0) / steps
    return env.max_over_ranks(s), int(hin.len), int(ho.len)


def run_ours(args):
    env = Env()
    pk = peaks()
    name = args.workload
    res = measure(env, name, args.steps, args.warmup)
    clocks = res.pop("clocks")
    info = res.pop("_info")
    ms = res["ms_per_step"]
    world = env.world

    if name.startswith("decode"):
        value, unit = info.get("bytes_total", world * info["bytes"]) / (ms * 1e-3) / 1e9, "GB/s"
        roof = {"bound": "hbm", "achieved": res["gbs_per_gpu"], "peak": float(pk["hbm_gbs"]), "unit": "GB/s", "frac": res["frac_of_hbm_peak"],
                "traffic": NCU_TRAFFIC.get(name), "peak_source": pk["_source"],
                "note": "per GPU; algorithmic bytes = 2*kv*Hkv*D*2 B a sequence x sequences a launch; duration = CUDA-event time of a step "
                        "(the split kernel plus its merge kernel)"}
        scaling = "strong" if "bytes_total" in info else "weak"
    elif name.startswith("mla_decode") or name.startswith("ds2_decode") or name.startswith("glm_sel"):
        value, unit = info.get("bytes_total", info["bytes"]) / (ms * 1e-3) / 1e9, "GB/s"
        roof = {"bound": "hbm", "achieved": res["gbs_per_gpu"], "peak": float(pk["hbm_gbs"]), "unit": "GB/s", "frac": res["frac_of_hbm_peak"],
                "traffic": NCU_TRAFFIC.get(name), "peak_source": pk["_source"], "note": "algorithmic bytes = 1,152 B a cell; flops 278,528 a cell",
                "tensor_frac": info["flops"] / (ms * 1e-3) / 1e12 / float(pk["bf16_tflops"])}
        scaling = "weak"
    else:
        value, unit = res.get("tflops_job", res["tflops_per_gpu"]), "TFLOP/s"
        roof = {"bound": "tensor", "achieved": res["tflops_per_gpu"], "peak": float(pk["bf16_tflops"]), "unit": "TFLOP/s",
                "frac": res["frac_of_bf16_peak"], "traffic": None, "peak_source": pk["_source"],
                "note": "per GPU; causal-exact flops (masked tiles not counted) / CUDA-event time; burst bf16 peak"}
        scaling = "strong"

    if args.kernel_only:
        if env.rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": unit, "n_gpus": world, "steps": res["steps"], "ms_per_step": ms,
                              "kernel_only": True, "config": config_of(name, world), "clocks": clocks}))
        env.close()
        return

    line = {
        "metric": METRIC, "value": value, "unit": unit, "n_gpus": world, "steps": res["steps"], "warmup": max(3, args.warmup), "ms_per_step": ms,
        "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "bf16" if name == "mla_prefill_c4" else "f16", "data": "synthetic",
        "config": config_of(name, world), "roofline": roof, "gpu_launches": int(res["steps"] * info["launches"]), "clocks": clocks,
    }
    if "check" in info:      # a workload that can check its own output (the multi-GPU exchanges): after the timed region
        line["parity"] = info["check"]()
    if "published" in res:
        line["published"] = res["published"]
    if name == "decode_c2":
        e2e_steps = max(5, min(args.steps, 200))
        # e2e: the batch through the library's batched C-ABI calls from pinned host buffers; beside it the same batch through
        # the reference's own per-sequence symbols (what an engine gets by swapping the library and changing nothing else)
        s2, h2d2, d2h2 = e2e_decode_native(env, info, e2e_steps)
        line["e2e"] = {"value": world * info["bytes"] / s2 / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d2, "d2h_bytes_per_step": d2h2,
                       "ms_per_step": s2 * 1e3,
                       "path": "one ns_copy_to of q (fp16) | k | v rows (one pinned buffer) -> one ns_b200_kv_store_batch -> one "
                               "ns_b200_gqa_decode for the batch -> one ns_copy_from out (fp16); ns_sync a step"}
        s, h2d, d2h = e2e_decode(env, info, e2e_steps)
        line["e2e_reference_symbols"] = {"value": world * info["bytes"] / s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                                         "ms_per_step": s * 1e3,
                                         "path": "per sequence: ns_copy_to q,k,v rows (pinned) -> ns_q35_kv_store -> ns_q35_attn_decode -> "
                                                 "ns_copy_from out; ns_sync a step"}
    del info, res

    if not args.no_others:
        others = {}
        for oname, osteps in (OTHERS_1GPU if world == 1 else OTHERS_NGPU):
            if oname == name:
                continue
            try:
                # every workload under its own clock record (a tensor-bound figure means little without the SM clock it ran
                # at), its timed region at least 100 ms long so that the record holds samples taken under its load
                r = measure(env, oname, osteps, 3, min_ms=100.0)
                oinfo = r.pop("_info")
                others[oname] = {k: (round(v, 4) if isinstance(v, float) else v) for k, v in r.items() if k != "workload"}
                if "check" in oinfo:
                    others[oname]["parity"] = oinfo["check"]()
                del oinfo
            except Exception as e:   # a failed extra must not take the headline with it
                others[oname] = {"error": str(e)[:200]}
        line["others"] = others

    if env.rank == 0:
        if world == 1 and not args.no_cpu:
            bps, cores, n, per = cpu_decode_rate(args.cpu_seconds)
            line["cpu_baseline"] = {"value": bps / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                                    "sample": f"one sequence of config 2 (134,217,728 KV bytes) x {n} repeats, {per * 1e3:.1f} ms each; "
                                              "CPU restatement of the reference decode kernel's numerics"}
        print(json.dumps(line))
    env.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_c2")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-others", action="store_true", help="skip the other configurations")
    ap.add_argument("--cpu-seconds", type=float, default=6.0)
    ap.add_argument("--kernel-only", action="store_true", help="device-timed headline only (no end-to-end, CPU or other legs): for profiler runs")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
