"""ns_b200_gqa_decode_static: split-KV decode for callers that cannot allocate (a memory plan fixed at load, a serving
loop that must not stall on cudaMalloc). Its partials live in an array inside the library; the result must equal the
entry point that takes caller scratch, and the CPU oracle. Runs last so that a failure here cannot hide another test's."""
import numpy as np
import pytest

from nextsycl_b200 import DevBuf
from nextsycl_b200 import workloads as W
from oracle import oracle as O

pytestmark = pytest.mark.gpu
ABS, REL = 2e-3, 1e-2


def _case(gpu, ops, seed, B, T, Hq, Hkv, D, kvs, cap):
    qs, seqs, keep, want = [], [], [], []
    for b, kv in enumerate(kvs):
        q, k, v, p0 = W.gqa_case(seed, T, Hq, Hkv, D, kv, cap=cap, seq=b)
        qs.append(q)
        dk, dv = DevBuf.of(gpu, k), DevBuf.of(gpu, v)
        keep += [dk, dv]
        seqs.append((dk, dv, cap, p0))
        want.append(O.gqa_flash_decode(q.astype(np.float32), k.view(np.uint16), v.view(np.uint16), T, Hq, Hkv, D, cap, p0))
    return DevBuf.of(gpu, np.stack(qs)), ops.seq_table(seqs), keep, np.stack(want).reshape(-1)


def test_static_scratch_decode_equals_caller_scratch_twice(gpu, ops):
    api = gpu.api
    f = api.need("ns_b200_gqa_decode_static")
    # two calls in a row per shape, different shapes; the second batch's shorter sequence needs more splits (37) than its
    # longest (36): the layout must hold for every length up to max_kv
    shapes = [(3, 2, 16, 2, 128, [700, 3000, 1234], 3008), (2, 1, 64, 8, 128, [9000, 4736], 9000)]
    for i, (B, T, Hq, Hkv, D, kvs, cap) in enumerate(shapes):
        dq, table, keep, oracle = _case(gpu, ops, 990 + i, B, T, Hq, Hkv, D, kvs, cap)
        n = B * T * Hq * D
        want = DevBuf(gpu, n * 2)
        sc = DevBuf(gpu, max(4, 4 * ops.gqa_decode_scratch(B, T, Hq, Hkv, D, max(kvs))))
        ops.gqa_decode(dq, Hq * D, T * Hq * D, table, B, T, Hq, Hkv, D, max(kvs), want, sc)
        w = want.read(np.float16).astype(np.float32)
        assert np.all(np.abs(w - oracle) <= ABS + REL * np.abs(oracle)), (i, "caller scratch vs oracle")
        got = DevBuf(gpu, n * 2)
        free_before = None
        for call in range(2):
            got.fill(0xFF)
            gpu.sync()
            if call == 1:
                free_before = gpu.memory()[1]   # the first call on a device did the one-time set-up; this one must allocate nothing
            rc = f(gpu.raw, dq.ptr, Hq * D, T * Hq * D, table.ptr, B, T, Hq, Hkv, D, max(kvs), got.ptr)
            assert rc == 0, api.last_error()
            gpu.sync()
            if call == 1:
                assert gpu.memory()[1] == free_before, "the call changed the device's free memory"
            o = got.read(np.float16).astype(np.float32)
            assert np.isfinite(o).all()
            assert np.all(np.abs(o - w) <= ABS + REL * np.abs(w)), (i, call, float(np.abs(o - w).max()))
            assert np.all(np.abs(o - oracle) <= ABS + REL * np.abs(oracle)), (i, call, "vs oracle")


def test_static_scratch_rejects_what_does_not_fit(gpu, ops):
    api = gpu.api
    d = DevBuf(gpu, 4096)
    # 64 sequences x 8 rows x 64 heads x 37 splits x 130 floats: far beyond 4 Mi floats
    rc = api.need("ns_b200_gqa_decode_static")(gpu.raw, d.ptr, 64 * 128, 8 * 64 * 128, d.ptr, 64, 8, 64, 8, 128, 32768, d.ptr)
    assert rc == -1
    assert "built-in scratch holds" in api.last_error()
    gpu.sync()
