"""One rank of the multi-GPU KV-split parity check (launched by tests/test_kvsplit_multigpu.py under torch.distributed.run,
one process a GPU). Every rank draws the same seeded context, keeps its own key range on its own GPU, runs a few steps
of split decode + push + combine, and checks the combined rows against the CPU oracle's decode of the whole context and
against every other rank's result (bit for bit: all ranks merge the same partials in the same order). Exits non-zero on a
mismatch."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from nextsycl_b200 import DevBuf, Gpu  # noqa: E402
from nextsycl_b200 import workloads as W  # noqa: E402
from nextsycl_b200.dist import KvSplit, key_ranges  # noqa: E402
from oracle import oracle as O  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", os.environ["RANK"]))
    dist.init_process_group("gloo")
    torch.cuda.set_device(local)
    gpu = Gpu(local)
    T, Hq, Hkv, D = 4, 32, 4, 128

    def exchange(h):
        out = [None] * world
        dist.all_gather_object(out, h)
        return out
    grp = KvSplit(gpu, rank, world, T, Hq, D, exchange=exchange)
    ok = True
    # a ragged context (the last rank's range is shorter), a context shorter than the ranks' shares (some ranks hold no
    # key and still publish), and the benchmark's long-context configuration at full size
    for kv in (20000 + 64 * 7, 70, 262144):
        ok = one_context(gpu, grp, rank, world, T, Hq, Hkv, D, kv) and ok
    ok = mla_context(gpu, rank, world, exchange, 131072) and ok
    grp.close()
    flags = [None] * world
    dist.all_gather_object(flags, ok)
    dist.destroy_process_group()
    if rank == 0:
        print("kvsplit multi-gpu:", "ok" if all(flags) else "MISMATCH", f"({world} ranks)", flush=True)
    sys.exit(0 if all(flags) else 1)


def mla_context(gpu, rank, world, exchange, n):
    """The absorbed-MLA latent cache (benchmark configuration 3 at 131,072 cells) split by cell ranges over the ranks: every
    rank's combined rows against the oracle on 16 heads spread over the tile, and against the other ranks' bit for bit."""
    T, H = 1, 128
    scale = float(1.0 / np.sqrt(192.0))
    q = W.normal_f16(3, 0, (T, H, 576))
    cache = W.normal_f16(3, 1, (n, 576), 0.5)
    grp = KvSplit(gpu, rank, world, T, H, 512, exchange=exchange)
    base, count = key_ranges(n, world)[rank]
    dq, dc = DevBuf.of(gpu, q), DevBuf.of(gpu, np.ascontiguousarray(cache[base:base + count]))
    sc = DevBuf(gpu, 4 * grp.mla_scratch_floats(count))
    out = DevBuf(gpu, T * H * 512 * 4)
    heads = [0, 31, 32, 63, 64, 95, 96, 127, 7, 16, 45, 50, 77, 88, 101, 120]
    box = [None]
    if rank == 0:
        O.use_all_cores()
        box[0] = O.mla_gemm(np.ascontiguousarray(q[:, heads].astype(np.float32)), cache.view(np.uint16), T, len(heads), 512, 64, n - T, np.float32(scale))
    dist.broadcast_object_list(box, src=0)
    want = box[0]
    ok = True
    for step in range(3):
        out.fill(0xFF)
        grp.mla_decode(dq, dc, count, base, n - T, scale, sc)
        grp.mla_combine(out)
        gpu.sync()
        got = out.read(np.float32).reshape(T, H, 512)
        d = np.abs(got[:, heads].astype(np.float64) - want)
        if not (np.isfinite(got).all() and np.all(d <= 2e-3 + 1e-2 * np.abs(want))):
            print(f"rank {rank} step {step} (MLA, {n} cells): max abs {d.max():.3e} outside |d| <= 2e-3 + 1e-2 |want|", flush=True)
            ok = False
        every = [None] * world
        dist.all_gather_object(every, got.tobytes())
        if any(e != every[0] for e in every):
            print(f"rank {rank} step {step} (MLA): the ranks' results differ", flush=True)
            ok = False
        dist.barrier()
    grp.close()
    if rank == 0:
        print(f"  MLA {n} cells over {world} ranks: {'ok' if ok else 'MISMATCH'}", flush=True)
    return ok


def one_context(gpu, grp, rank, world, T, Hq, Hkv, D, kv):
    q, k, v, p0 = W.gqa_case(5, T, Hq, Hkv, D, kv)
    base, count = key_ranges(kv, world)[rank]
    dq = DevBuf.of(gpu, q)
    dk = DevBuf.of(gpu, np.ascontiguousarray(k[:, base:base + count])) if count else None
    dv = DevBuf.of(gpu, np.ascontiguousarray(v[:, base:base + count])) if count else None
    scratch = DevBuf(gpu, 4 * grp.scratch_floats(Hkv, count)) if count else None
    out = DevBuf(gpu, T * Hq * D * 2)
    # the whole context's decode on the CPU: rank 0 computes it on every core it may use and hands it round
    box = [None]
    if rank == 0:
        O.use_all_cores()
        box[0] = O.gqa_flash_decode(q.astype(np.float32), k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, kv, p0)
    dist.broadcast_object_list(box, src=0)
    want = box[0]
    del k, v
    ok = True
    for step in range(5):
        out.fill(0xFF)
        if step < 3:
            grp.decode(dq, Hq * D, dk, dv, Hkv, count, base, p0, scratch)
            grp.combine(out)
        else:
            grp.step(dq, Hq * D, dk, dv, Hkv, count, base, p0, scratch, out)    # the same step as one kernel launch
        gpu.sync()
        got = out.read(np.float16).reshape(T, Hq * D)
        d = np.abs(got.astype(np.float64) - want)
        if not (np.isfinite(got).all() and np.all(d <= 2e-3 + 1e-2 * np.abs(want))):
            print(f"rank {rank} step {step} ({kv} keys): max abs {d.max():.3e} outside |d| <= 2e-3 + 1e-2 |want|", flush=True)
            ok = False
        every = [None] * world
        dist.all_gather_object(every, got.view(np.uint16).tobytes())
        if any(e != every[0] for e in every):
            print(f"rank {rank} step {step}: the ranks' results differ", flush=True)
            ok = False
        dist.barrier()
    if rank == 0:
        print(f"  {kv} keys over {world} ranks: {'ok' if ok else 'MISMATCH'}", flush=True)
    return ok


if __name__ == "__main__":
    main()
