"""The KV-split decode across ranks.

CPU part: the partition of a context into key ranges, and the handle exchange over torch.distributed (gloo, 2 ranks).
GPU part (one GPU): all ranks' slices run one after another on the same stream, each pushing into every rank's
mailbox, then each rank's combine - by then every flag is set, so nothing ever waits on another launch. A combine whose
peer never published gives up its bounded wait and the next sync reports it."""
import os
import subprocess
import sys

import numpy as np
import pytest

from nextsycl_b200.dist import key_ranges

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_key_ranges_cover_the_context():
    for kv, n in [(262144, 8), (262144, 1), (1000, 4), (100, 8), (65, 2), (64, 2)]:
        r = key_ranges(kv, n)
        assert len(r) == n and r[0][0] == 0
        assert sum(c for _, c in r) == kv
        for (b0, c0), (b1, _) in zip(r, r[1:]):
            assert b1 == b0 + c0
            assert b1 % 64 == 0 or b1 == kv
    assert key_ranges(262144, 8)[3] == (98304, 32768)


GLOO_SCRIPT = r"""
import os, sys
sys.path.insert(0, %r)
import torch.distributed as dist
from nextsycl_b200.dist import key_ranges
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%%s" %% sys.argv[1], rank=int(sys.argv[2]), world_size=2)
rank = dist.get_rank()
handle = bytes([rank]) * 64
got = [None, None]
dist.all_gather_object(got, handle)
assert got[0] == bytes([0]) * 64 and got[1] == bytes([1]) * 64
base, count = key_ranges(1000, 2)[rank]
assert (base, count) == ((0, 512) if rank == 0 else (512, 488))
dist.barrier()
dist.destroy_process_group()
print("ok", rank)
"""


def test_handle_exchange_over_gloo(tmp_path):
    script = tmp_path / "gloo_ranks.py"
    script.write_text(GLOO_SCRIPT % ROOT)
    port = str(29500 + os.getpid() % 2000)
    procs = [subprocess.Popen([sys.executable, str(script), port, str(r)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    for p in procs:
        out, err = p.communicate(timeout=120)
        assert p.returncode == 0, err
        assert out.startswith("ok")


@pytest.mark.gpu
@pytest.mark.parametrize("nranks,T,Hq,Hkv,kv", [(2, 1, 16, 2, 1000), (4, 4, 32, 4, 5000), (8, 4, 32, 4, 20000), (3, 2, 8, 2, 130),
                                                  (8, 1, 8, 2, 100),      # six of the eight ranks hold no key at all
                                                  (2, 4, 32, 4, 9537)])   # the last rank holds 4,737 keys: its rows 0..2 see <= 4,736 and need 74 splits, not 38
def test_all_ranks_on_one_gpu_match_the_oracle(gpu, ops, nranks, T, Hq, Hkv, kv):
    from nextsycl_b200 import DevBuf
    from nextsycl_b200 import workloads as W
    from nextsycl_b200.dist import KvSplit
    from oracle import oracle as O
    D = 128
    q, k, v, p0 = W.gqa_case(950, T, Hq, Hkv, D, kv)
    dq = DevBuf.of(gpu, q)
    nbytes = KvSplit.mailbox_bytes(gpu.api, nranks, T, Hq, D)
    boxes = [DevBuf(gpu, nbytes) for _ in range(nranks)]
    for b in boxes:
        b.fill(0)
    groups = [KvSplit(gpu, r, nranks, T, Hq, D, local_mailboxes=boxes) for r in range(nranks)]
    want = O.gqa_flash_decode(q.astype(np.float32), k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, kv, p0)
    keep = []
    for step in range(2):   # two steps: both mailbox buffers, and the counter's return to zero
        for r, (base, count) in enumerate(key_ranges(kv, nranks)):
            if count == 0:
                # a rank past the end of a short context still publishes (an empty partial), with no caches and no scratch
                groups[r].decode(dq, Hq * D, None, None, Hkv, 0, base, p0, None)
                continue
            dk, dv = DevBuf.of(gpu, np.ascontiguousarray(k[:, base:base + count])), DevBuf.of(gpu, np.ascontiguousarray(v[:, base:base + count]))
            sc = DevBuf(gpu, 4 * groups[r].scratch_floats(Hkv, count))
            sc.fill(0xFF)
            keep += [dk, dv, sc]
            groups[r].decode(dq, Hq * D, dk, dv, Hkv, count, base, p0, sc)
        for r in range(nranks):
            out = DevBuf(gpu, T * Hq * D * 2)
            out.fill(0xFF)
            groups[r].combine(out, wait_us=1000)
            gpu.sync()
            got = out.read(np.float16).reshape(T, Hq * D).astype(np.float32)
            d = np.abs(got - want)
            assert np.all(d <= 2e-3 + 1e-2 * np.abs(want)), (step, r, float(d.max()))


@pytest.mark.gpu
def test_combine_gives_up_when_a_peer_never_publishes(gpu, ops):
    from nextsycl_b200 import DevBuf, Error
    from nextsycl_b200.dist import KvSplit
    T, Hq, D, nranks = 1, 8, 128, 2
    boxes = [DevBuf(gpu, KvSplit.mailbox_bytes(gpu.api, nranks, T, Hq, D)) for _ in range(nranks)]
    for b in boxes:
        b.fill(0)
    g0 = KvSplit(gpu, 0, nranks, T, Hq, D, local_mailboxes=boxes)
    out = DevBuf(gpu, T * Hq * D * 2)
    g0.combine(out, epoch=1, wait_us=2000)      # nobody published epoch 1
    with pytest.raises(Error, match="bounded wait"):
        gpu.sync()
    gpu.sync()                                   # the report clears; the context stays usable
    assert DevBuf.of(gpu, np.arange(4, dtype=np.float32)).read(np.float32).sum() == 6


@pytest.mark.gpu
def test_recorded_step_replays_with_device_epochs(gpu, ops):
    """One rank's step (slice decode + push + combine) recorded with ns_q35_graph_begin/end and replayed: the step number
    lives in the mailbox, so every replay is a new epoch on alternating buffers."""
    from nextsycl_b200 import DevBuf
    from nextsycl_b200 import workloads as W
    from nextsycl_b200.dist import KvSplit
    from oracle import oracle as O
    T, Hq, Hkv, D, kv = 4, 32, 4, 128, 3000
    q, k, v, p0 = W.gqa_case(951, T, Hq, Hkv, D, kv)
    dq, dk, dv = DevBuf.of(gpu, q), DevBuf.of(gpu, k), DevBuf.of(gpu, v)
    box = DevBuf(gpu, KvSplit.mailbox_bytes(gpu.api, 1, T, Hq, D))
    box.fill(0)
    grp = KvSplit(gpu, 0, 1, T, Hq, D, local_mailboxes=[box])
    sc = DevBuf(gpu, 4 * grp.scratch_floats(Hkv, kv))
    out = DevBuf(gpu, T * Hq * D * 2)

    def one():
        grp.decode(dq, Hq * D, dk, dv, Hkv, kv, 0, p0, sc, epoch=0)
        grp.combine(out, epoch=0, wait_us=1000)
    one()                      # first call outside any recording (it sets kernel attributes)
    gpu.sync()
    graph = gpu.record(one)
    want = O.gqa_flash_decode(q.astype(np.float32), k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, kv, p0)
    for rep in range(3):
        out.fill(0xFF)
        graph.launch()
        gpu.sync()
        got = out.read(np.float16).reshape(T, Hq * D).astype(np.float32)
        assert np.all(np.abs(got - want) <= 2e-3 + 1e-2 * np.abs(want)), rep
    graph.free()


@pytest.mark.gpu
@pytest.mark.parametrize("T,Hq,Hkv,D,kv", [(4, 32, 4, 128, 3000), (1, 64, 8, 128, 20000), (2, 24, 4, 256, 900), (8, 16, 1, 128, 5000)])
def test_the_step_as_one_kernel(gpu, ops, T, Hq, Hkv, D, kv):
    """ns_b200_kvsplit_step with one rank (its own mailbox is the only one): split decode, merge, push, flag, poll and combine
    inside one cooperative launch, called twice and then replayed from a recording (step numbers on the device). The last
    shape (128 rows of one key head: four row groups x 296 splits) does not fit the GPU at once and takes the three launches."""
    from nextsycl_b200 import DevBuf
    from nextsycl_b200 import workloads as W
    from nextsycl_b200.dist import KvSplit
    from oracle import oracle as O
    q, k, v, p0 = W.gqa_case(952, T, Hq, Hkv, D, kv)
    dq, dk, dv = DevBuf.of(gpu, q), DevBuf.of(gpu, k), DevBuf.of(gpu, v)
    box = DevBuf(gpu, KvSplit.mailbox_bytes(gpu.api, 1, T, Hq, D))
    box.fill(0)
    grp = KvSplit(gpu, 0, 1, T, Hq, D, local_mailboxes=[box])
    sc = DevBuf(gpu, 4 * grp.scratch_floats(Hkv, kv))
    sc.fill(0xFF)
    out = DevBuf(gpu, T * Hq * D * 2)
    want = O.gqa_flash_decode(q.astype(np.float32), k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, kv, p0)

    def one():
        grp.step(dq, Hq * D, dk, dv, Hkv, kv, 0, p0, sc, out, epoch=0, wait_us=100000)

    def check(what):
        gpu.sync()
        got = out.read(np.float16).reshape(T, Hq * D).astype(np.float32)
        assert np.isfinite(got).all(), what
        assert np.all(np.abs(got - want) <= 2e-3 + 1e-2 * np.abs(want)), (what, float(np.abs(got - want).max()))
    for i in range(2):
        out.fill(0xFF)
        one()
        check(f"call {i}")
    graph = gpu.record(one)
    for rep in range(3):
        out.fill(0xFF)
        graph.launch()
        check(f"replay {rep}")
    graph.free()


@pytest.mark.gpu
def test_partials_gathered_by_the_caller(gpu, ops):
    """ns_b200_kvsplit_partial per key range, the partials laid side by side as an all-gather would leave them,
    ns_b200_kvsplit_merge: the library-exchange baseline's two ends."""
    from nextsycl_b200 import DevBuf
    from nextsycl_b200 import workloads as W
    from nextsycl_b200.core import check
    from oracle import oracle as O
    api = gpu.api
    nranks, T, Hq, Hkv, D, kv = 4, 4, 32, 4, 128, 7000
    q, k, v, p0 = W.gqa_case(953, T, Hq, Hkv, D, kv)
    dq = DevBuf.of(gpu, q)
    rows = T * Hq
    parts = DevBuf(gpu, nranks * rows * (D + 2) * 4)
    parts.fill(0xFF)
    keep = []
    for r, (base, count) in enumerate(key_ranges(kv, nranks)):
        dk, dv = DevBuf.of(gpu, np.ascontiguousarray(k[:, base:base + count])), DevBuf.of(gpu, np.ascontiguousarray(v[:, base:base + count]))
        sc = DevBuf(gpu, 4 * int(api.ns_b200_kvsplit_scratch(T, Hq, Hkv, D, count)))
        keep += [dk, dv, sc]
        check(api, api.ns_b200_kvsplit_partial(gpu.raw, dq.ptr, Hq * D, dk.ptr, dv.ptr, T, Hq, Hkv, D, count, base, p0, sc.ptr,
                                               parts.ptr + r * rows * (D + 2) * 4), "partial")
    out = DevBuf(gpu, rows * D * 2)
    check(api, api.ns_b200_kvsplit_merge(gpu.raw, parts.ptr, nranks, T, Hq, D, out.ptr), "merge")
    gpu.sync()
    got = out.read(np.float16).reshape(T, Hq * D).astype(np.float32)
    want = O.gqa_flash_decode(q.astype(np.float32), k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, kv, p0)
    assert np.all(np.abs(got - want) <= 2e-3 + 1e-2 * np.abs(want)), float(np.abs(got - want).max())


@pytest.mark.gpu
@pytest.mark.parametrize("nranks,T,H,n", [(2, 1, 128, 1000), (4, 3, 128, 5000), (8, 1, 128, 20000), (3, 2, 16, 130), (8, 1, 128, 100)])
def test_mla_cell_ranges_on_one_gpu_match_the_oracle(gpu, ops, nranks, T, H, n):
    """The absorbed-MLA latent cache split by cell ranges: every rank's slice run one after another on one GPU, each pushing
    into every rank's mailbox, then each rank's combine (all flags set by then: nothing waits on another launch). Against the
    oracle's decode of the whole cache; two steps (both mailbox buffers). (8 ranks over 100 cells: six hold none.)"""
    from nextsycl_b200 import DevBuf
    from nextsycl_b200 import workloads as W
    from nextsycl_b200.dist import KvSplit
    from oracle import oracle as O
    scale = float(1.0 / np.sqrt(192.0))
    q = W.normal_f16(955, 0, (T, H, 576))
    cache = W.normal_f16(955, 1, (n, 576), 0.5)
    pos0 = n - T
    dq = DevBuf.of(gpu, q)
    boxes = [DevBuf(gpu, KvSplit.mailbox_bytes(gpu.api, nranks, T, H, 512)) for _ in range(nranks)]
    for b in boxes:
        b.fill(0)
    groups = [KvSplit(gpu, r, nranks, T, H, 512, local_mailboxes=boxes) for r in range(nranks)]
    want = O.mla_gemm(q.astype(np.float32), cache.view(np.uint16), T, H, 512, 64, pos0, np.float32(scale))
    keep = []
    for step in range(2):
        for r, (base, count) in enumerate(key_ranges(n, nranks)):
            if count == 0:
                groups[r].mla_decode(dq, None, 0, base, pos0, scale, None)
                continue
            dc = DevBuf.of(gpu, np.ascontiguousarray(cache[base:base + count]))
            sc = DevBuf(gpu, 4 * groups[r].mla_scratch_floats(count))
            sc.fill(0xFF)
            keep += [dc, sc]
            groups[r].mla_decode(dq, dc, count, base, pos0, scale, sc)
        for r in range(nranks):
            out = DevBuf(gpu, T * H * 512 * 4)
            out.fill(0xFF)
            groups[r].mla_combine(out, wait_us=1000)
            gpu.sync()
            got = out.read(np.float32).reshape(T, H, 512)
            d = np.abs(got - want)
            assert np.isfinite(got).all() and np.all(d <= 2e-3 + 1e-2 * np.abs(want)), (step, r, float(d.max()))


@pytest.mark.gpu
def test_the_one_kernel_step_refuses_a_step_number_whose_tag_is_zero(gpu, ops):
    from nextsycl_b200 import DevBuf
    api = gpu.api
    d = DevBuf(gpu, 1 << 20)
    rc = api.ns_b200_kvsplit_step(gpu.raw, d.ptr, 128, d.ptr, d.ptr, 1, 1, 1, 128, 64, 0, 63, d.ptr, 0, 1, d.ptr, d.ptr, 1 << 32, 1000, d.ptr)
    assert rc == -1 and "low 32 bits" in api.last_error()
    gpu.sync()
